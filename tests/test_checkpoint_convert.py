"""Converted Hugging Face Llama weights reproduce the HF model's logits; TP/PP split and merge are inverse."""
import pytest
import torch

from megatron_lm_b200.checkpoint import convert


def test_hf_llama_logits_match(tmp_path):
    transformers = pytest.importorskip("transformers")
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    torch.manual_seed(0)
    hc = transformers.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                  rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False,
                                  attn_implementation="eager")
    hf = transformers.LlamaForCausalLM(hc).eval()
    sd = convert.hf_llama_to_core(hf.state_dict(), 2, 4, 2)
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2,
                            ffn_hidden_size=112, normalization="RMSNorm", gated_linear_unit=True,
                            activation_func="silu", add_bias_linear=False, hidden_dropout=0.0, attention_dropout=0.0,
                            layernorm_epsilon=1e-5)
    m = GPTModel(cfg, 96, 64, position_embedding_type="rope", share_embeddings_and_output_weights=False,
                 parallel_output=False).eval()
    missing = m.load_state_dict(sd, strict=False)
    assert not [k for k in missing.missing_keys if "_extra_state" not in k], missing
    ids = torch.randint(0, 96, (2, 17))
    with torch.no_grad():
        ours = m(ids)
        theirs = hf(ids).logits
    assert torch.allclose(ours, theirs, atol=2e-4, rtol=1e-3), (ours - theirs).abs().max()
    back = convert.core_to_hf_llama(m.state_dict(), 2, 4, 2)
    for k, v in hf.state_dict().items():
        if k in back:
            assert torch.equal(back[k], v), k
    # repartition: tp 2 x pp 2 and back
    stages = convert.split_for_pp(sd, 2, 2)
    parts = [convert.split_for_tp(st, 2) for st in stages]
    assert parts[0][0]["decoder.layers.0.mlp.linear_fc1.weight"].shape == (112, 64)
    merged = convert.merge_pp([convert.merge_tp(p) for p in parts])
    for k, v in sd.items():
        assert torch.equal(merged[k], v), k
    convert.save_core(parts, str(tmp_path), 0, {"num_layers": 2})
    again = convert.load_core(str(tmp_path))
    assert all(torch.equal(again[k], v) for k, v in sd.items())
    legacy = convert.core_to_legacy(sd)
    assert "language_model.encoder.layers.1.self_attention.query_key_value.weight" in legacy
    assert set(convert.legacy_to_core(legacy)) == set(sd)
