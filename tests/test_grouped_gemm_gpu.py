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
