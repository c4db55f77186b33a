"""FP8 quantisation and GEMM: CPU emulation invariants; GPU kernels against the emulation / fp32."""
import pytest
import torch

from megatron_lm_b200.ops.fp8 import (gemm_fp8, linear_fp8, mxfp8_dequantize, mxfp8_quantize, quantize)


def test_quantize_roundtrip_cpu():
    torch.manual_seed(0)
    x = torch.randn(64, 96) * 3
    q = quantize(x, 0)
    assert q.data.shape == (64, 96) and q.data_t.shape == (96, 64)
    err = (q.dequantize() - x).abs().max() / x.abs().max()
    assert err < 0.07                                   # e4m3: 3 mantissa bits
    assert torch.equal(q.data_t, q.data.t())
    z = quantize(torch.zeros(16, 16), 0)
    assert float(z.scale_inv) == 1.0


def test_mxfp8_roundtrip_cpu():
    torch.manual_seed(0)
    x = torch.randn(64, 128) * torch.logspace(-3, 3, 128)
    for rows in (True, False):
        q, s = mxfp8_quantize(x, rows)
        back = mxfp8_dequantize(q, s, rows)
        rel = ((back - x).abs() / (x.abs() + 1e-9)).median()
        assert rel < 0.05


def test_linear_fp8_cpu_close_to_fp32():
    torch.manual_seed(0)
    x = torch.randn(32, 64, requires_grad=True)
    w = torch.randn(48, 64, requires_grad=True) * 0.1
    w.retain_grad()
    y = linear_fp8(x, w, None, "hybrid")
    ref = x @ w.t()
    assert (y - ref).abs().max() / ref.abs().max() < 0.08
    y.sum().backward()
    assert x.grad.shape == x.shape and w.grad.shape == w.shape
    assert (w.grad - torch.ones(32, 48).t() @ x.detach()).abs().max() / w.grad.abs().max() < 0.1


@pytest.mark.gpu
def test_fp8_kernels_gpu():
    torch.manual_seed(0)
    x = (torch.randn(256, 512, device="cuda") * 2).bfloat16()
    q = quantize(x, 0)
    qc = quantize(x.cpu(), 0)
    assert torch.allclose(q.scale_inv.cpu(), qc.scale_inv, rtol=1e-6)
    # bit-exact except for ties broken differently by the two roundings of x * scale
    mism = (q.data.cpu() != qc.data).float().mean()
    assert mism < 0.01, mism
    assert torch.equal(q.data_t, q.data.t().contiguous())
    q5 = quantize(x, 1)
    assert (q5.dequantize() - x.float()).abs().max() / x.float().abs().max() < 0.13
    for M, N, K in ((256, 384, 512), (128, 128, 144), (512, 1024, 4096)):
        a = (torch.randn(M, K, device="cuda")).bfloat16()
        b = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
        aq, bq = quantize(a, 0, False), quantize(b, 0, False)
        ref = aq.dequantize() @ bq.dequantize().t()
        out = gemm_fp8(aq.data, 0, aq.scale_inv, bq.data, 0, bq.scale_inv)
        assert torch.allclose(out.float(), ref, atol=2e-2 * ref.abs().max().item(), rtol=2e-2), (M, N, K)
        acc = torch.ones(M, N, device="cuda")
        gemm_fp8(aq.data, 0, aq.scale_inv, bq.data, 0, bq.scale_inv, out=acc, accumulate=True)
        assert torch.allclose(acc, ref + 1, atol=1e-3 * ref.abs().max().item() + 1e-3, rtol=1e-3)
    # mixed e5m2 x e4m3, as in the gradient products
    g = torch.randn(256, 384, device="cuda").bfloat16()
    w = (torch.randn(384, 512, device="cuda") * 0.05).bfloat16()
    gq, wq = quantize(g, 1, False), quantize(w.t().contiguous(), 0, False)
    out = gemm_fp8(gq.data, 1, gq.scale_inv, wq.data, 0, wq.scale_inv)
    ref = gq.dequantize() @ wq.dequantize().t()
    assert torch.allclose(out.float(), ref, atol=2e-2 * ref.abs().max().item(), rtol=2e-2)
    # the autograd linear against fp32
    xx = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ww = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    ww.main_grad = torch.zeros(384, 256, device="cuda")
    y = linear_fp8(xx, ww, None, "hybrid")
    gy = torch.randn_like(y)
    y.backward(gy)
    ry = xx.float() @ ww.float().t()
    assert (y.float() - ry).abs().max() / ry.abs().max() < 0.1
    rgw = gy.float().t() @ xx.float()
    assert (ww.main_grad - rgw).abs().max() / rgw.abs().max() < 0.15
    rgx = gy.float() @ ww.float()
    assert (xx.grad.float() - rgx).abs().max() / rgx.abs().max() < 0.15
    # MXFP8
    xm = torch.randn(128, 256, device="cuda").bfloat16()
    for rows in (True, False):
        qg, sg = mxfp8_quantize(xm, rows)
        qc_, sc_ = mxfp8_quantize(xm.cpu(), rows)
        assert torch.equal(sg.cpu(), sc_)
        assert (qg.cpu() != qc_).float().mean() < 0.01


def test_model_with_fp8_config_cpu():
    """``fp8='hybrid'`` routes layer linears through the FP8 path (emulated on CPU) and still trains."""
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    torch.manual_seed(0)
    kw = dict(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128, hidden_dropout=0.0,
              attention_dropout=0.0, params_dtype=torch.bfloat16, bf16=True, add_bias_linear=False)
    m8 = GPTModel(TransformerConfig(fp8="hybrid", fp8_recipe="tensorwise", **kw), 64, 32)
    torch.manual_seed(0)
    m16 = GPTModel(TransformerConfig(**kw), 64, 32)
    ids = torch.randint(0, 64, (2, 16))
    l8, l16 = m8(ids, labels=ids).mean(), m16(ids, labels=ids).mean()
    assert abs(float(l8) - float(l16)) < 0.05 and float(l8) != float(l16)
    l8.backward()
    g = m8.decoder.layers[0].mlp.linear_fc1.weight.grad
    assert g is not None and torch.isfinite(g.float()).all()


def test_first_and_last_layers_can_stay_in_16_bits():
    import torch
    from megatron_lm_b200 import fp8_utils as F8
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.transformer import TransformerBlock
    cfg = TransformerConfig(num_layers=4, hidden_size=32, num_attention_heads=4, fp8="hybrid", first_last_layers_bf16=True,
                            num_layers_at_start_in_bf16=1, num_layers_at_end_in_bf16=2)
    assert [F8.layer_runs_in_fp8(cfg, i) for i in range(4)] == [False, True, False, False]
    blk = TransformerBlock(cfg)
    marks = [getattr(l.mlp.linear_fc1, "fp8_eligible", True) for l in blk.layers]
    assert marks == [False, True, False, False]
    assert all(getattr(l.self_attention.linear_qkv, "fp8_eligible", True) == m for l, m in zip(blk.layers, marks))
    with F8.get_fp8_context(cfg, 0):
        assert cfg.fp8 is None
    with F8.get_fp8_context(cfg, 1):
        assert cfg.fp8 == "hybrid"
    assert cfg.fp8 == "hybrid"
    assert F8.get_fp8_align_size("mxfp8") == 32 and F8.get_fp8_align_size("delayed") == 16
    t = torch.zeros(2, dtype=torch.float8_e4m3fn)
    assert F8.is_float8tensor(t) and not F8.is_float8tensor(torch.zeros(2))


# ----------------------------------------------------------------------------- block-scaled (MXFP8) tensor-core GEMM
def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()

def _mx_ref(a, b):
    return a.dequantize().float() @ b.dequantize().float().t()


def test_mx_dual_quantiser_cpu_roundtrip():
    from megatron_lm_b200.ops import fp8
    torch.manual_seed(0)
    x = torch.randn(96, 160) * 3
    r, c = fp8.mxfp8_quantize_dual(x)
    assert r.data.shape == (96, 160) and c.data.shape == (160, 96)
    assert r.sf.numel() == fp8.mx_sf_bytes(96, 160) and c.sf.numel() == fp8.mx_sf_bytes(160, 96)
    # e4m3 keeps 3 mantissa bits: relative error of a block-scaled value stays under 2^-3 of the block maximum
    assert (r.dequantize() - x).abs().max() <= 0.0625 * x.abs().max()
    assert (c.dequantize() - x.t()).abs().max() <= 0.0625 * x.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(64, 128), (256, 384), (4096, 1024), (96, 160)])
def test_mx_dual_quantiser_matches_cpu(rows, cols):
    from megatron_lm_b200.ops import fp8
    torch.manual_seed(1)
    x = (torch.randn(rows, cols) * 2).to(torch.bfloat16)
    rc, cc = fp8.mxfp8_quantize_dual(x)
    rg, cg = fp8.mxfp8_quantize_dual(x.cuda())
    assert torch.equal(rg.data.cpu(), rc.data) and torch.equal(cg.data.cpu(), cc.data)
    idx_r = fp8.mx_sf_index(rows, cols).reshape(-1)
    idx_c = fp8.mx_sf_index(cols, rows).reshape(-1)
    assert torch.equal(rg.sf.cpu()[idx_r], rc.sf[idx_r]) and torch.equal(cg.sf.cpu()[idx_c], cc.sf[idx_c])


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 192, 128), (256, 384, 256), (512, 256, 512), (300, 200, 96), (1024, 1000, 4096),
                                   (4096, 4096, 1024)])
def test_mx_gemm_matches_dequantised_product(M, N, K):
    """The tensor core applies the 1 x 32 scales itself: the result must equal the fp32 product of the dequantised
    operands (same quantised inputs on both sides, so only accumulation order differs)."""
    from megatron_lm_b200.ops import _lib, fp8
    torch.manual_seed(2)
    # rows with very different magnitudes, so a wrong scale byte (row or K-block mix-up) shows at once
    A = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 2, M, device="cuda").unsqueeze(1)).to(torch.bfloat16)
    B = (torch.randn(N, K, device="cuda") * (1 + torch.arange(K, device="cuda") // 32 % 7).unsqueeze(0)).to(torch.bfloat16)
    a, _ = fp8.mxfp8_quantize_dual(A, colwise=False)
    b, _ = fp8.mxfp8_quantize_dual(B, colwise=False)
    ref = _mx_ref(a, b)
    out32 = fp8.gemm_mx(a, b, out_dtype=torch.float32)
    out16 = fp8.gemm_mx(a, b, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(out32, ref) < 1e-5 * K ** 0.5
    assert torch.allclose(out32, ref, rtol=1e-3, atol=1e-3 * ref.abs().max().item())
    assert _rel(out16, ref) < 1e-2
    acc = torch.ones(M, N, device="cuda")
    fp8.gemm_mx(a, b, out=acc, accumulate=True)
    assert _rel(acc, ref + 1) < 1e-5 * K ** 0.5


@pytest.mark.gpu
def test_mx_linear_gradients_close_to_bf16():
    from megatron_lm_b200.ops import _lib, fp8
    torch.manual_seed(3)
    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.nn.Parameter(torch.randn(384, 256, device="cuda", dtype=torch.bfloat16) * 0.1)
    y = fp8.linear_mxfp8(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(dy.float())
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(y, yr) < 6e-2 and _rel(x.grad, xr.grad) < 8e-2 and _rel(w.grad, wr.grad) < 8e-2
