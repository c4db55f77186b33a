"""Post-training quantisation: number formats, calibration, smoothing recipes, compressed weights, state round trip,
tensor-parallel range agreement.  The reference tests the same flow through an external library
(tests/unit_tests/post_training/test_modelopt_module_spec.py, tests/unit_tests/inference/test_modelopt_gpt_model.py)."""
import copy
import json

import pytest
import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.gpt import GPTModel
from megatron_lm_b200.post_training import ptq
from tests.dist_utils import run_distributed


def _model(seed=0, hidden=64, ffn=128):
    torch.manual_seed(seed)
    cfg = TransformerConfig(num_layers=2, hidden_size=hidden, num_attention_heads=4, ffn_hidden_size=ffn,
                            hidden_dropout=0.0, attention_dropout=0.0, gated_linear_unit=True, add_bias_linear=False)
    m = GPTModel(cfg, 96, 32, parallel_output=False)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.08)
    return cfg, m


def _batch(n=4, s=32, seed=1):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 96, (n, s), generator=g)
    return ids, torch.arange(s).unsqueeze(0).expand(n, s)


def _logits(m, ids, pos):
    with torch.no_grad():
        return m(ids, pos, None).float()


def test_number_formats_round_trip_on_their_grids():
    x = torch.tensor([[0.0, 0.4, -0.6, 1.2, 1.6, -2.4, 3.6, 5.1, 6.0, -7.0, 0.2, 0.3, 0.74, 0.76, 2.6, -3.4]])
    q = ptq.fake_quant(x, ptq.QuantizerSpec("nvfp4", block=(1, 16)), torch.tensor(6.0))
    # block range 7 -> block scale 7/6 rounded to E4M3 (1.125 * ... ) ; every output is a grid value times the scale
    scale = (q.abs().max() / 6.0).item()
    grid = torch.tensor(ptq._E2M1_GRID) * scale
    assert all((grid - v.abs()).abs().min() < 1e-6 for v in q.flatten())
    assert (q - x).abs().max() <= 0.5 * scale + 1e-6 + 1.0 * scale      # coarse top steps of E2M1
    w = torch.randn(130, 70)
    for spec in (ptq.QuantizerSpec("fp8"), ptq.QuantizerSpec("fp8", block=(128, 128)),
                 ptq.QuantizerSpec("int8", axis=0), ptq.QuantizerSpec("int4", block=(1, 128))):
        amax = w.abs().amax(dim=1) if spec.axis == 0 else w.abs().amax()
        q = ptq.fake_quant(w, spec, amax)
        assert q.shape == w.shape
        rel = ((q - w).norm() / w.norm()).item()
        assert rel < {"fp8": 0.04, "int8": 0.01, "int4": 0.15}[spec.kind], (spec, rel)
        assert torch.allclose(ptq.fake_quant(q, spec, amax), q, atol=1e-5)            # a second pass changes nothing
    # int8 per-tensor: exactly 255 levels
    q = ptq.fake_quant(w, ptq.QuantizerSpec("int8"), w.abs().amax())
    assert q.unique().numel() <= 255


@pytest.mark.parametrize("fmt,tol", [("fp8", 0.15), ("fp8_blockwise", 0.15), ("fp8_blockwise_32", 0.15),
                                     ("int8_sq", 0.06), ("int4_awq", 0.45), ("w4a8_awq", 0.45), ("nvfp4", 0.5)])
def test_quantize_calibrates_and_stays_close(fmt, tol):
    cfg, m = _model()
    ids, pos = _batch()
    ref = _logits(m, ids, pos)
    names = ptq.quantize(m, fmt, lambda mod: mod(ids, pos, None))
    assert len(names) == 2 * 4 and not any("output_layer" in n for n in names)
    lin = m.decoder.layers[0].mlp.linear_fc1
    assert lin.ptq and lin.input_quantizer.sample is None and not lin.input_quantizer.calibrating
    if fmt in ("fp8", "int8_sq", "w4a8_awq", "nvfp4"):
        assert lin.input_quantizer.amax is not None and lin.input_quantizer.amax.numel() == 1
    if fmt in ("int8_sq", "int4_awq", "w4a8_awq"):
        assert lin.input_quantizer._pre_quant_scale.shape == (cfg.hidden_size,)
    out = _logits(m, ids, pos)
    rel = ((out - ref).norm() / ref.norm()).item()
    assert 0 < rel < tol, (fmt, rel)
    ptq.disable_quantizers(m)
    if fmt not in ("int8_sq", "int4_awq", "w4a8_awq"):        # folding changed the weights of the smoothing recipes
        assert torch.equal(_logits(m, ids, pos), ref)
    ptq.enable_quantizers(m)
    assert torch.equal(_logits(m, ids, pos), out)


def test_smoothing_preserves_the_unquantised_function_and_helps_outliers():
    cfg, m = _model(seed=3)
    ids, pos = _batch(seed=5)
    # an activation outlier channel: scale one embedding column up, and the weights that read it down
    with torch.no_grad():
        m.decoder.layers[0].self_attention.linear_qkv.weight[:, 7] *= 0.02
        m.decoder.layers[0].input_layernorm.weight[7] *= 50.0
    ref = _logits(m, ids, pos)
    plain = copy.deepcopy(m)
    plain_names = ptq.attach_quantizers(plain, "int8_sq")
    mods = dict(plain.named_modules())
    for n in plain_names:
        mods[n].input_quantizer.calibrating = True
    plain(ids, pos, None)
    ptq._finish_calibration(plain, plain_names, None)          # same formats, no smoothing
    err_plain = (_logits(plain, ids, pos) - ref).norm()
    ptq.quantize(m, "int8_sq", lambda mod: mod(ids, pos, None))
    err_sq = (_logits(m, ids, pos) - ref).norm()
    assert err_sq < err_plain
    # with the quantisers in pass-through mode the folded model computes the original function
    for _, lin in ptq.quantized_linears(m):
        if lin.ptq:
            lin.input_quantizer.spec.enabled = lin.weight_quantizer.spec.enabled = False
    assert torch.allclose(_logits(m, ids, pos), ref, atol=2e-4, rtol=1e-4)


def test_straight_through_gradient_reaches_the_weights():
    cfg, m = _model()
    ids, pos = _batch(2)
    ptq.quantize(m, "fp8", lambda mod: mod(ids, pos, None))
    m(ids, pos, None).float().pow(2).mean().backward()
    g = m.decoder.layers[1].mlp.linear_fc2.weight.grad
    assert g is not None and torch.isfinite(g).all() and g.abs().sum() > 0


@pytest.mark.parametrize("fmt", ["fp8_real_quant", "fp8_blockwise_real_quant"])
def test_compressed_weights_and_state_round_trip(fmt, tmp_path):
    cfg, m = _model()
    ids, pos = _batch()
    ref = _logits(m, ids, pos)
    ptq.quantize(m, fmt, lambda mod: mod(ids, pos, None))
    lin = m.decoder.layers[0].mlp.linear_fc1
    assert lin.weight is None and lin.weight_q.dtype == torch.float8_e4m3fn
    if "blockwise" in fmt:
        assert lin.weight_scale.shape == (2 * 128 // 128, 1)          # [2*ffn / 128, hidden / 128 rounded up]
    out = _logits(m, ids, pos)
    assert ((out - ref).norm() / ref.norm()).item() < 0.15
    assert not any(n.endswith("linear_fc1.weight") for n, _ in m.named_parameters())
    # structure description + state dict load into a freshly built model
    state = json.loads(json.dumps(ptq.quantizer_state(m)))
    torch.save(m.state_dict(), tmp_path / "q.pt")
    _, fresh = _model(seed=9)
    ptq.restore_quantizer_state(fresh, state)
    missing, unexpected = fresh.load_state_dict(torch.load(tmp_path / "q.pt"), strict=False)
    assert not unexpected and not [k for k in missing if "_extra_state" not in k]
    assert torch.equal(_logits(fresh, ids, pos), out)


def test_compress_reports_bytes():
    cfg, m = _model()
    ids, pos = _batch(2)
    ptq.quantize(m, "fp8", lambda mod: mod(ids, pos, None))
    r = ptq.compress(m)
    n = sum(l.weight_q.numel() for _, l in ptq.quantized_linears(m) if l.ptq)
    assert r["before"] == 4 * n and r["after"] == n + 4 * 8            # fp32 test model -> one byte + one scale each


def _tp_rank(rank, world):
    from megatron_lm_b200.parallel import state
    from tests.model_utils import reinit_by_global_name
    state.initialize_model_parallel(tensor_model_parallel_size=2)
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, add_bias_linear=False)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(3))
    pos = torch.arange(16).unsqueeze(0).expand(2, 16)
    for fmt in ("fp8", "int8_sq"):
        mm = GPTModel(cfg, 64, 16, parallel_output=False)
        reinit_by_global_name(mm, cfg)
        ptq.quantize(mm, fmt, lambda mod: mod(ids, pos, None))
        for name, lin in ptq.quantized_linears(mm):
            if not lin.ptq:
                continue
            vals = [lin.input_quantizer.amax.clone()]
            if lin.weight_quantizer.spec.axis is None:
                vals.append(lin.weight_quantizer.amax.clone())
            if fmt == "int8_sq" and "linear_qkv" in name or "linear_fc1" in name and fmt == "int8_sq":
                vals.append(lin.input_quantizer._pre_quant_scale.clone())
            for v in vals:
                got = [torch.zeros_like(v) for _ in range(world)]
                torch.distributed.all_gather(got, v)
                assert torch.equal(got[0], got[1]), (fmt, name)
        out = mm(ids, pos, None)
        assert torch.isfinite(out).all()


def test_ranges_agree_across_tensor_parallel_ranks():
    run_distributed(_tp_rank, 2)


_FLAGS = ["--num-layers", "2", "--hidden-size", "64", "--num-attention-heads", "4", "--seq-length", "32",
          "--max-position-embeddings", "32", "--micro-batch-size", "2", "--tokenizer-type", "NullTokenizer",
          "--vocab-size", "95", "--distributed-backend", "gloo", "--use-cpu-initialization",
          "--attention-dropout", "0", "--hidden-dropout", "0", "--swiglu", "--disable-bias-linear",
          "--normalization", "RMSNorm", "--position-embedding-type", "rope", "--untie-embeddings-and-output-weights",
          "--calib-size", "8", "--calib-batch-size", "4", "--mock-data"]


def _program_rank(rank, world, out_dir, fmt):
    import os
    from megatron_lm_b200.post_training.checkpointing import STATE_FILE
    from megatron_lm_b200.tasks import quantize_gpt
    from megatron_lm_b200.training import checkpointing
    from megatron_lm_b200.training.arguments import get_args
    argv = _FLAGS + ["--tensor-model-parallel-size", str(world), "--save", out_dir, "--export-quant-cfg", fmt,
                     "--export-qk-l2-norm"]
    res = quantize_gpt.main(argv)
    assert res["linears"] == 8 and res["before"] > 1.0 and abs(res["after"] / res["before"] - 1.0) < 0.2
    rank_dir = os.path.join(out_dir, "iter_0000001", f"mp_rank_{rank:02d}")
    assert os.path.isfile(os.path.join(rank_dir, STATE_FILE))
    # a freshly built model picks the quantisers up from the checkpoint
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.training.arguments import core_transformer_config_from_args
    args = get_args()
    cfg = core_transformer_config_from_args(args)
    cfg.qk_l2_norm = True
    fresh = GPTModel(cfg, vocab_size=args.padded_vocab_size, max_sequence_length=32, parallel_output=True,
                     share_embeddings_and_output_weights=False, position_embedding_type="rope")
    args.load = out_dir
    checkpointing.load_checkpoint([fresh], None, None, args)
    lin = fresh.decoder.layers[1].mlp.linear_fc2
    assert lin.ptq and lin.input_quantizer.amax is not None and float(lin.input_quantizer.amax) > 0
    if fmt.endswith("real_quant"):
        assert lin.weight is None and lin.weight_q.dtype == torch.float8_e4m3fn
    batches = list(quantize_gpt.calibration_batches(args))
    assert abs(quantize_gpt.perplexity(fresh.eval(), batches, torch.device("cpu")) - res["after"]) < 1e-3 * res["after"]


@pytest.mark.parametrize("world,fmt", [(1, "fp8_real_quant"), (2, "int8_sq")])
def test_calibration_program_saves_a_loadable_quantised_model(world, fmt, tmp_path):
    run_distributed(_program_rank, world, str(tmp_path / "q"), fmt)


@pytest.mark.gpu
def test_compressed_weights_feed_the_fp8_gemm_directly():
    """On a GPU the per-tensor FP8 weights go to the FP8 tensor-core GEMM as stored; the result matches the
    de-quantise-then-multiply path up to the activation cast."""
    dev = torch.device("cuda")
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=2, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512,
                            hidden_dropout=0.0, attention_dropout=0.0, gated_linear_unit=True, add_bias_linear=False,
                            params_dtype=torch.bfloat16, bf16=True)
    m = GPTModel(cfg, 96, 64, parallel_output=False).to(dev)
    ids = torch.randint(0, 96, (4, 64), device=dev)
    pos = torch.arange(64, device=dev).unsqueeze(0).expand(4, 64)
    ref = _logits(m, ids, pos)
    ptq.quantize(m, "fp8_real_quant", lambda mod: mod(ids, pos, None))
    before = ptq.FAST_PATH_CALLS[0]
    fast = _logits(m, ids, pos)
    assert ptq.FAST_PATH_CALLS[0] - before == 8                     # every compressed linear took the FP8 GEMM
    for _, lin in ptq.quantized_linears(m):
        lin.ptq_dequantize_only = True
    slow = _logits(m, ids, pos)
    assert ptq.FAST_PATH_CALLS[0] - before == 8
    assert ((fast - slow).norm() / slow.norm()).item() < 0.05
    assert ((fast - ref).norm() / ref.norm()).item() < 0.15
