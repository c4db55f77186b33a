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


def test_mamba_tensor_parallel_repartition_round_trip_and_layout():
    """A Mamba mixer's in_proj / conv segments are re-cut per segment: splitting an unpartitioned state dict to 2 ranks
    gives each rank [z_r | x_r | B_r | C_r | dt_r], and merging returns the original."""
    import torch
    from megatron_lm_b200.checkpoint.convert import mamba_merge_tp, mamba_split_for_tp
    torch.manual_seed(0)
    d_model, nheads, headdim, ngroups, d_state, d_conv = 32, 8, 8, 4, 16, 4
    d_inner = nheads * headdim
    rows = 2 * d_inner + 2 * ngroups * d_state + nheads
    sd = {"decoder.layers.0.mixer.in_proj.weight": torch.randn(rows, d_model),
          "decoder.layers.0.mixer.conv_weight": torch.randn(d_inner + 2 * ngroups * d_state, d_conv),
          "decoder.layers.0.mixer.conv_bias": torch.randn(d_inner + 2 * ngroups * d_state),
          "decoder.layers.0.mixer.dt_bias": torch.randn(nheads), "decoder.layers.0.mixer.A_log": torch.randn(nheads),
          "decoder.layers.0.mixer.D": torch.randn(nheads), "decoder.layers.0.mixer.norm_weight": torch.randn(d_inner),
          "decoder.layers.0.mixer.out_proj.weight": torch.randn(d_model, d_inner),
          "decoder.layers.0.norm.weight": torch.randn(d_model),
          "decoder.layers.1.mlp.linear_fc1.weight": torch.randn(2 * 48, d_model),
          "decoder.layers.1.mlp.linear_fc2.weight": torch.randn(d_model, 48),
          "embedding.word_embeddings.weight": torch.randn(64, d_model)}
    parts = mamba_split_for_tp(sd, 2, nheads, ngroups, d_state)
    w = sd["decoder.layers.0.mixer.in_proj.weight"]
    z, x, B, C, dt = torch.split(w, [d_inner, d_inner, ngroups * d_state, ngroups * d_state, nheads], dim=0)
    for r in range(2):
        want = torch.cat([t.chunk(2, 0)[r] for t in (z, x, B, C, dt)], 0)
        assert torch.equal(parts[r]["decoder.layers.0.mixer.in_proj.weight"], want)
        assert parts[r]["decoder.layers.0.mixer.conv_weight"].shape[0] == (d_inner + 2 * ngroups * d_state) // 2
        assert parts[r]["decoder.layers.0.mixer.out_proj.weight"].shape == (d_model, d_inner // 2)
        assert torch.equal(parts[r]["decoder.layers.0.norm.weight"], sd["decoder.layers.0.norm.weight"])
        assert parts[r]["decoder.layers.1.mlp.linear_fc1.weight"].shape[0] == 48
    back = mamba_merge_tp(parts, nheads, ngroups, d_state)
    assert back.keys() == sd.keys()
    for k in sd:
        assert torch.equal(back[k], sd[k]), k
    four = mamba_split_for_tp(back, 4, nheads, ngroups, d_state)
    assert torch.equal(mamba_merge_tp(four, nheads, ngroups, d_state)["decoder.layers.0.mixer.in_proj.weight"], w)


def test_mamba_repartitioned_weights_run_a_mixer():
    """The split layout is the one the mixer computes with: a TP1 mixer and its re-cut weights give the same in_proj
    segments a TP2 rank would slice out."""
    import torch
    from megatron_lm_b200.checkpoint.convert import mamba_split_for_tp
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.mamba import MambaMixer
    torch.manual_seed(1)
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4)
    m = MambaMixer(cfg, 1, d_state=16, headdim=8, ngroups=4)
    sd = {"decoder.layers.0.mixer." + k: v.detach() for k, v in m.state_dict().items()}
    parts = mamba_split_for_tp(sd, 2, m.nheads, m.ngroups, m.d_state)
    x = torch.randn(5, 1, 32)
    full = torch.nn.functional.linear(x, sd["decoder.layers.0.mixer.in_proj.weight"])
    z, xs, B, C, dt = torch.split(full, [m.d_inner, m.d_inner, m.ngroups * m.d_state, m.ngroups * m.d_state, m.nheads], -1)
    for r in range(2):
        loc = torch.nn.functional.linear(x, parts[r]["decoder.layers.0.mixer.in_proj.weight"])
        want = torch.cat([t.chunk(2, -1)[r] for t in (z, xs, B, C, dt)], -1)
        assert torch.allclose(loc, want, atol=1e-6)


def test_hf_mixtral_round_trip_and_logits(tmp_path):
    """HF Mixtral -> core -> HF is the identity, and the core weights reproduce the HF model's logits."""
    import pytest
    import torch
    transformers = pytest.importorskip("transformers")
    from megatron_lm_b200.checkpoint.convert import core_to_hf_mixtral, hf_llama_to_core
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    torch.manual_seed(0)
    hcfg = transformers.MixtralConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, num_local_experts=4,
                                      num_experts_per_tok=2, max_position_embeddings=64, rope_theta=10000.0,
                                      rms_norm_eps=1e-5, tie_word_embeddings=False, router_jitter_noise=0.0)
    hf_model = transformers.MixtralForCausalLM(hcfg).eval()
    hf_sd = {k: v.detach().clone() for k, v in hf_model.state_dict().items()}
    core = hf_llama_to_core(hf_sd, 2, 4, 2)
    back = core_to_hf_mixtral(core, 2, 4, 2)            # checkpoint-file names: block_sparse_moe.experts.<e>.w1 / w3 / w2
    again = hf_llama_to_core(back, 2, 4, 2)
    assert again.keys() == core.keys()
    for k, v in core.items():
        assert torch.equal(v, again[k]), k
    if "model.layers.0.mlp.experts.gate_up_proj" in hf_sd:
        gu = hf_sd["model.layers.0.mlp.experts.gate_up_proj"]
        assert torch.equal(back["model.layers.0.block_sparse_moe.experts.1.w1.weight"], gu[1][:96])
        assert torch.equal(back["model.layers.0.block_sparse_moe.experts.1.w3.weight"], gu[1][96:])
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=96,
                            moe_ffn_hidden_size=96, num_moe_experts=4, moe_router_topk=2, normalization="RMSNorm",
                            layernorm_epsilon=1e-5, gated_linear_unit=True, activation_func="silu", add_bias_linear=False,
                            hidden_dropout=0.0, attention_dropout=0.0, moe_aux_loss_coeff=0.0)
    model = GPTModel(cfg, vocab_size=128, max_sequence_length=64, position_embedding_type="rope",
                     share_embeddings_and_output_weights=False).eval()
    missing, unexpected = model.load_state_dict(core, strict=False)
    assert not unexpected, unexpected
    assert all("_extra_state" in m or "rotary" in m for m in missing), missing
    tokens = torch.randint(0, 128, (2, 16))
    with torch.no_grad():
        ours = model(tokens).transpose(0, 1) if model(tokens).shape[0] == 16 else model(tokens)
        ref = hf_model(tokens).logits
    assert torch.allclose(ours.float(), ref.float(), atol=2e-4, rtol=1e-3), (ours - ref).abs().max()


def test_hf_llava_round_trip_and_logits(tmp_path):
    """HF LLaVA (CLIP tower, second-to-last layer features without the class token, two-layer projector, Llama) ->
    core ``LLaVAModel`` reproduces the library's logits; core -> HF -> core is the identity; the command line reads a
    Hugging Face directory and writes tensor-parallel core shards."""
    import json
    import pytest
    import torch
    transformers = pytest.importorskip("transformers")
    from megatron_lm_b200.checkpoint import convert
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.multimodal import LLaVAModel
    torch.manual_seed(0)
    v = transformers.CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=2,
                                      image_size=28, patch_size=14, hidden_act="quick_gelu", layer_norm_eps=1e-5)
    t = transformers.LlamaConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                 num_key_value_heads=2, vocab_size=128, max_position_embeddings=64, rms_norm_eps=1e-5,
                                 rope_theta=10000.0, tie_word_embeddings=False)
    hcfg = transformers.LlavaConfig(vision_config=v, text_config=t, image_token_index=127, vision_feature_layer=-2,
                                    vision_feature_select_strategy="default", projector_hidden_act="gelu",
                                    image_seq_length=4)
    hf_model = transformers.LlavaForConditionalGeneration(hcfg).eval()
    hf_sd = {k: p.detach().clone() for k, p in hf_model.state_dict().items()}
    kw = dict(num_layers=2, num_heads=4, num_query_groups=2, vision_layers=2, vision_heads=2)
    core = convert.hf_llava_to_core(hf_sd, **kw)
    back = convert.core_to_hf_llava(core, patch_dim=14, **kw)
    again = convert.hf_llava_to_core(back, **kw)
    assert again.keys() == core.keys() and all(torch.equal(core[k], again[k]) for k in core)
    for k, p in back.items():                                  # everything LLaVA reads is restored bit for bit
        if "encoder.layers.2." not in k and "post_layernorm" not in k:
            assert torch.equal(p, hf_sd[k]), k
    files = convert.core_to_hf_llava(core, patch_dim=14, in_memory_names=False, **kw)   # names of the released files
    assert "language_model.model.layers.0.self_attn.q_proj.weight" in files and "language_model.lm_head.weight" in files
    assert all(torch.equal(core[k], x) for k, x in convert.hf_llava_to_core(files, **kw).items())
    lcfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=96,
                             normalization="RMSNorm", layernorm_epsilon=1e-5, gated_linear_unit=True,
                             activation_func="silu", add_bias_linear=False, hidden_dropout=0.0, attention_dropout=0.0)
    vcfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=2, ffn_hidden_size=64,
                             activation_func="quick_gelu", layernorm_epsilon=1e-5, hidden_dropout=0.0,
                             attention_dropout=0.0)
    pcfg = TransformerConfig(num_layers=1, hidden_size=64, num_attention_heads=4, ffn_hidden_size=64,
                             activation_func="gelu", hidden_dropout=0.0, attention_dropout=0.0)
    model = LLaVAModel(lcfg, 128, 64, vcfg, pcfg, drop_vision_class_token=True, img_h=28, img_w=28, patch_dim=14,
                       language_position_embedding_type="rope", image_token_index=127, parallel_output=False).eval()
    missing, unexpected = model.load_state_dict(core, strict=False)
    assert not unexpected and all("_extra_state" in m or "rotary" in m for m in missing), (missing, unexpected)
    images = torch.randn(2, 3, 28, 28)
    ids = torch.randint(0, 120, (2, 12))
    hf_ids = ids.clone()
    hf_ids[:, 2:6] = 127                                       # the library wants one placeholder per image embedding
    our_ids = torch.cat([ids[:, :2], torch.full((2, 1), 127), ids[:, 6:]], dim=1)   # ours splices at a single token
    with torch.no_grad():
        ref = hf_model(input_ids=hf_ids, pixel_values=images).logits
        out = model(images, our_ids)
    out = out if out.shape[0] == 2 else out.transpose(0, 1)
    assert out.shape == ref.shape
    assert torch.allclose(out.float(), ref.float(), atol=3e-4, rtol=1e-3), (out - ref).abs().max()
    # command line: HF directory in, two tensor-parallel core shards out (vision MLP cut as a plain MLP)
    hf_dir, out_dir = tmp_path / "hf", tmp_path / "core"
    hf_dir.mkdir()
    torch.save(files, hf_dir / "pytorch_model.bin")
    (hf_dir / "config.json").write_text(json.dumps({
        "text_config": {"num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "hidden_size": 64,
                        "intermediate_size": 96, "vocab_size": 128},
        "vision_config": {"num_hidden_layers": 3, "num_attention_heads": 2, "patch_size": 14, "image_size": 28},
        "vision_feature_layer": -2, "image_token_index": 127}))
    convert.main(["--loader", "llava_hf", "--saver", "core", "--load-dir", str(hf_dir), "--save-dir", str(out_dir),
                  "--target-tensor-parallel-size", "2"])
    r0 = torch.load(out_dir / "release" / "mp_rank_00" / "model_optim_rng.pt", weights_only=False)["model"]
    r1 = torch.load(out_dir / "release" / "mp_rank_01" / "model_optim_rng.pt", weights_only=False)["model"]
    fc1 = core["vision_model.decoder.layers.0.mlp.linear_fc1.weight"]
    assert torch.equal(torch.cat([r0["vision_model.decoder.layers.0.mlp.linear_fc1.weight"],
                                  r1["vision_model.decoder.layers.0.mlp.linear_fc1.weight"]]), fc1)
    g = core["language_model.decoder.layers.0.mlp.linear_fc1.weight"]
    assert torch.equal(r1["language_model.decoder.layers.0.mlp.linear_fc1.weight"], torch.cat([g[48:96], g[144:192]]))
