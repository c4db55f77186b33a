"""tcgen05 GEMM against an fp32 PyTorch product, all operand layouts and output modes."""
import pytest
import torch

from megatron_lm_b200.ops import _lib
from megatron_lm_b200.ops.gemm import gemm, linear

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 128, 192), (200, 328, 136),
                                   (4096, 4096, 1024), (77, 40, 72)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need the contiguous dim to be a multiple of 8")
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(out, ref) < 1e-2
    # element-level check on a sample (catches swizzle / descriptor mistakes that keep norms close)
    assert torch.allclose(out.float(), ref, atol=0.5, rtol=5e-2)


@pytest.mark.parametrize("dynamic", [False, True])
@pytest.mark.parametrize("M,N,K", [(300, 520, 200), (257, 264, 72), (512, 300, 136), (1000, 32000, 256),
                                   (4096, 11008, 4096), (4096, 4096, 11008), (4096, 32000, 4096)])
def test_gemm_pair_kernel_ragged_and_model_shapes(M, N, K, dynamic):
    """Shapes that reach the CTA-pair kernel (M, N >= 256): ragged edges, the vocabulary projection, the MLP
    products of the 7B model; with the static and with the dynamic (counter-drawn) tile schedule."""
    from megatron_lm_b200.ops import gemm as G
    torch.manual_seed(5)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    old = G._DYNAMIC
    G._DYNAMIC = dynamic
    try:
        for _ in range(2):                      # the second launch finds the schedule words back at zero
            out = gemm(A, B)
        # MN-major operands need their contiguous dim to be a multiple of 8
        wg = gemm(A, B.t().contiguous(), b_mn=True, out_dtype=torch.float32) if N % 8 == 0 else None
    finally:
        G._DYNAMIC = old
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(out, ref) < 1e-2
    assert torch.allclose(out.float(), ref, atol=0.05 * K ** 0.5, rtol=5e-2)
    if wg is not None:
        assert _rel(wg, ref) < 1e-4 * K ** 0.5


def test_gemm_dynamic_schedule_with_part_of_the_gpu_held():
    """Another stream holds 40 SMs for 0.2 s; the dynamic schedule finishes the product meanwhile."""
    from megatron_lm_b200.ops import gemm as G
    from megatron_lm_b200.ops.tp_fused import occupy_sms
    torch.manual_seed(6)
    A = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    old = G._DYNAMIC
    G._DYNAMIC = True
    try:
        gemm(A, B)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        occupy_sms(40, 200 * 1024, 200000, side)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(4):
            out = gemm(A, B)
        e1.record()
        torch.cuda.synchronize()
    finally:
        G._DYNAMIC = old
    _lib.check_status()
    assert e0.elapsed_time(e1) < 100.0, e0.elapsed_time(e1)
    assert _rel(out, ref) < 1e-2


def test_gemm_fp32_out_and_accumulate():
    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    out = gemm(A, B, out_dtype=torch.float32)
    assert _rel(out, ref) < 1e-5 * K ** 0.5
    base = torch.randn(M, N, device="cuda", dtype=torch.float32)
    acc = base.clone()
    gemm(A, B, out=acc, accumulate=True)
    assert _rel(acc, base + ref) < 1e-5 * K ** 0.5
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ob = gemm(A, B, bias=bias)
    assert _rel(ob, ref + bias.float()) < 1e-2
    _lib.check_status()


def test_gemm_fp16():
    torch.manual_seed(2)
    A = torch.randn(256, 128, device="cuda", dtype=torch.float16)
    B = torch.randn(384, 128, device="cuda", dtype=torch.float16)
    out = gemm(A, B)
    assert _rel(out, A.float() @ B.float().t()) < 2e-3


def test_linear_autograd_matches_reference():
    torch.manual_seed(3)
    x = torch.randn(64, 4, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = linear(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(dy.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2
    assert _rel(b.grad, br.grad) < 1e-2


def test_linear_accumulates_into_main_grad():
    torch.manual_seed(4)
    x = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    w = torch.nn.Parameter(torch.randn(384, 128, device="cuda", dtype=torch.bfloat16))
    w.main_grad = torch.zeros(384, 128, device="cuda", dtype=torch.float32)
    fired = []
    w.grad_ready = lambda: fired.append(1)
    for _ in range(2):
        linear(x, w).backward(torch.ones(256, 384, device="cuda", dtype=torch.bfloat16))
    ref = 2 * (torch.ones(256, 384, device="cuda") .t() @ x.float())
    assert w.grad is None and len(fired) == 2
    assert _rel(w.main_grad, ref) < 1e-3
