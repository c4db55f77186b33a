"""Grouped (ragged) expert GEMM in one launch against per-expert fp32 products: forward, dgrad, wgrad."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("splits,out_f,in_f", [([100, 0, 300, 129], 256, 192), ([128, 128], 384, 128),
                                               ([5, 7, 1, 0, 260, 3, 90, 64], 128, 320)])
def test_grouped_linear_matches_reference(splits, out_f, in_f):
    from megatron_lm_b200.ops.grouped_gemm import grouped_linear
    torch.manual_seed(0)
    E, T = len(splits), sum(splits)
    x = torch.randn(T, in_f, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(E, out_f, in_f, device="cuda") * 0.05).bfloat16().requires_grad_()
    w.main_grad = torch.zeros(E, out_f, in_f, device="cuda")
    y = grouped_linear(x, w, splits)
    gy = torch.randn_like(y)
    y.backward(gy)
    o = 0
    for e, n in enumerate(splits):
        xe, ge = x.detach()[o:o + n].float(), gy[o:o + n].float()
        ref = xe @ w.detach()[e].float().t()
        if n:
            assert torch.allclose(y[o:o + n].float(), ref, atol=2e-2, rtol=2e-2), (e, n)
            assert torch.allclose(x.grad[o:o + n].float(), ge @ w.detach()[e].float(), atol=2e-2, rtol=2e-2), (e, n)
        assert torch.allclose(w.main_grad[e], ge.t() @ xe, atol=5e-2, rtol=2e-2), (e, n)
        o += n


@pytest.mark.parametrize("splits,out_f,in_f", [([100, 0, 300, 129], 256, 192), ([64, 1, 63, 65, 0, 0, 200, 7], 128, 320),
                                               ([700, 1300], 1024, 512)])
@pytest.mark.parametrize("main_grad", [True, False])
def test_grouped_linear_with_device_side_splits(splits, out_f, in_f, main_grad):
    """Token counts stay on the device: tile table, tile count and expert offsets come from a kernel, the weight
    gradient of all experts is one launch (an expert's last reduction step is cut at its boundary; experts
    without tokens get a zero gradient)."""
    from megatron_lm_b200.ops import _lib
    from megatron_lm_b200.ops.grouped_gemm import grouped_linear
    torch.manual_seed(1)
    E, T = len(splits), sum(splits)
    x = torch.randn(T, in_f, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(E, out_f, in_f, device="cuda") * 0.05).bfloat16().requires_grad_()
    if main_grad:
        w.main_grad = torch.full((E, out_f, in_f), 0.5, device="cuda")
    counts = torch.tensor(splits, device="cuda", dtype=torch.int64)
    y = grouped_linear(x, w, counts)
    gy = torch.randn_like(y)
    y.backward(gy)
    torch.cuda.synchronize()
    _lib.check_status()
    gw = w.main_grad - 0.5 if main_grad else w.grad.float()
    o = 0
    for e, n in enumerate(splits):
        xe, ge = x.detach()[o:o + n].float(), gy[o:o + n].float()
        if n:
            assert torch.allclose(y[o:o + n].float(), xe @ w.detach()[e].float().t(), atol=2e-2, rtol=2e-2), (e, n)
            assert torch.allclose(x.grad[o:o + n].float(), ge @ w.detach()[e].float(), atol=2e-2, rtol=2e-2), (e, n)
        assert torch.allclose(gw[e], ge.t() @ xe, atol=6e-2, rtol=2e-2), (e, n, (gw[e] - ge.t() @ xe).abs().max())
        o += n
