import math

import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.export.trtllm import TRTLLMHelper
from megatron_lm_b200.models.gpt import GPTModel
from megatron_lm_b200.post_training.distillation import (HiddenStateCosineLoss, LogitsAndIntermediatesLossBalancer,
                                                         LogitsKLLoss)
from megatron_lm_b200.post_training.quant_config import RecipeConfig, apply_recipe
from megatron_lm_b200.tasks.zeroshot_gpt import LMDataset, evaluate, results, wikitext_detokenizer


def _m():
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, gated_linear_unit=True, add_bias_linear=False)
    return cfg, GPTModel(cfg, 64, 32, parallel_output=False)


def test_zeroshot_perplexity_counts_each_token_once():
    cfg, m = _m()
    toks = torch.randint(0, 64, (70,)).tolist()
    full = LMDataset(toks, 16, 0, 60, 70)
    over = LMDataset(toks, 16, 0, 60, 70, overlapping_eval=4)
    assert sum(int(full[i]["pad_mask"].sum()) for i in range(len(full))) == 69
    assert sum(int(over[i]["pad_mask"].sum()) for i in range(len(over))) == 69
    tot = evaluate(m, torch.utils.data.DataLoader(full, batch_size=2))
    r = results("WIKITEXT103", tot, full)
    assert abs(r["ppl"] - math.exp(tot / 69)) < 1e-6 and r["adjusted ppl"] > r["ppl"]
    assert wikitext_detokenizer("a @-@ b , c") == "a-b, c"


def test_trtllm_names():
    cfg, m = _m()
    h = TRTLLMHelper(cfg, "llama")
    w = h.convert(m.state_dict(), torch.float32)
    assert w["transformer.layers.0.attention.qkv.weight"].shape == (96, 32)
    assert w["transformer.layers.1.mlp.gate.weight"].shape == (64, 32)
    assert "lm_head.weight" in w and h.pretrained_config(vocab_size=64)["num_hidden_layers"] == 2


def test_distillation_losses_and_recipe():
    s, t = torch.randn(4, 3, 16, requires_grad=True), torch.randn(4, 3, 16)
    kl = LogitsKLLoss(temperature=2.0)(s, t)
    ref = torch.nn.functional.kl_div(torch.log_softmax(s / 2, -1), torch.softmax(t / 2, -1), reduction="none").sum(-1) * 4
    assert torch.allclose(kl, ref, atol=1e-5)
    assert float(LogitsKLLoss()(t, t).abs().max()) < 1e-6
    cos = HiddenStateCosineLoss(16, 16)(s, s.detach())
    assert float(cos.abs().max()) < 1e-6
    bal = LogitsAndIntermediatesLossBalancer(kd_loss_scale=1.0)
    out = bal({"original": torch.tensor(2.0), "logits_kl": torch.tensor(0.5), "hidden": torch.tensor(4.0)})
    assert abs(float(out) - 4.0) < 1e-5            # KD part rescaled to the original loss' magnitude
    cfg, m = _m()
    rec = RecipeConfig.from_config_dict({"matchers": {"a": {"pattern": "*layers.0.*", "config": "bf16"},
                                                      "b": {"pattern": "*", "config": "fp8"}},
                                         "configs": {"bf16": {"fp8": False}, "fp8": {"fp8": True}}})
    chosen = apply_recipe(m, rec)
    assert chosen["decoder.layers.0.mlp.linear_fc1"] == "bf16" and chosen["decoder.layers.1.mlp.linear_fc1"] == "fp8"
    assert m.decoder.layers[0].mlp.linear_fc1.fp8_eligible is False


def test_trtllm_rank_files_and_fp8_scales(tmp_path):
    import json
    import os
    from megatron_lm_b200.post_training import ptq
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=4, hidden_size=32, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, gated_linear_unit=True, add_bias_linear=False)
    m = GPTModel(cfg, 64, 32, parallel_output=False, share_embeddings_and_output_weights=False)
    h = TRTLLMHelper(cfg, "llama")
    full = h.convert(m.state_dict(), torch.float32)
    ranks = h.split_for_mapping(full, tp=2, pp=2)
    assert len(ranks) == 4
    # pipeline: two layers per stage, renumbered from zero; embedding first, head and final norm last
    assert "transformer.vocab_embedding.weight" in ranks[0] and "transformer.vocab_embedding.weight" not in ranks[2]
    assert "lm_head.weight" in ranks[3] and "transformer.ln_f.weight" in ranks[2] and "lm_head.weight" not in ranks[0]
    assert set(k.split(".")[2] for k in ranks[2] if k.startswith("transformer.layers.")) == {"0", "1"}
    # tensor: QKV by heads, so that every rank holds [its q ; its k ; its v]
    qkv = full["transformer.layers.2.attention.qkv.weight"]                       # [32 q + 16 k + 16 v, 32]
    r0, r1 = ranks[2]["transformer.layers.0.attention.qkv.weight"], ranks[3]["transformer.layers.0.attention.qkv.weight"]
    assert r0.shape == (32, 32)
    assert torch.equal(r1, torch.cat((qkv[16:32], qkv[40:48], qkv[56:64])))
    assert torch.equal(torch.cat((ranks[2]["transformer.layers.0.mlp.proj.weight"],
                                  ranks[3]["transformer.layers.0.mlp.proj.weight"]), 1),
                       full["transformer.layers.2.mlp.proj.weight"])
    assert ranks[1]["transformer.layers.1.mlp.gate.weight"].shape == (32, 32) and ranks[3]["lm_head.weight"].shape == (32, 32)
    with __import__("pytest").raises(ValueError):
        h.split_for_mapping(full, tp=3)
    files = h.save_checkpoint(str(tmp_path / "ck"), ranks, h.pretrained_config(tp=2, pp=2, vocab_size=64))
    assert len(files) == 4 and all(os.path.isfile(f) for f in files)
    assert json.load(open(tmp_path / "ck" / "config.json"))["mapping"] == {"world_size": 4, "tp_size": 2, "pp_size": 2}
    # FP8 scales of a calibrated model
    ids = torch.randint(0, 64, (2, 16))
    pos = torch.arange(16).unsqueeze(0).expand(2, 16)
    ptq.quantize(m, "fp8", lambda mod: mod(ids, pos, None))
    sc = h.fp8_scaling_factors(m)
    lin = m.decoder.layers[1].mlp.linear_fc1
    assert torch.allclose(sc["transformer.layers.1.mlp.fc.weights_scaling_factor"], lin.weight_quantizer.amax / 448.0)
    assert torch.equal(sc["transformer.layers.1.mlp.gate.activation_scaling_factor"],
                       sc["transformer.layers.1.mlp.fc.activation_scaling_factor"])
    assert len(sc) == 4 * (4 * 2 + 2)
    # per-expert modules become one stacked tensor
    moe_cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                                num_moe_experts=4, moe_ffn_hidden_size=48, gated_linear_unit=True, add_bias_linear=False,
                                moe_grouped_gemm=False)
    moe = GPTModel(moe_cfg, 64, 32, parallel_output=False)
    w = TRTLLMHelper(moe_cfg, "mixtral").convert(moe.state_dict(), torch.float32)
    assert w["transformer.layers.0.mlp.fc.weight"].shape == (4, 96, 32) and w["transformer.layers.0.mlp.proj.weight"].shape == (4, 32, 48)
