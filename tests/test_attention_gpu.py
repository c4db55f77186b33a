"""tcgen05 flash attention (forward + backward) against the fp32 PyTorch body."""
import math

import pytest
import torch

from megatron_lm_b200.ops import _lib
from megatron_lm_b200.ops.attention import _ref_attention, attention, fused_qkv_attention

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("s,b,ng,qpg,d", [(128, 1, 1, 1, 128), (256, 2, 2, 1, 128), (384, 1, 2, 2, 64),
                                          (200, 1, 1, 2, 128), (1024, 1, 4, 1, 128), (640, 1, 1, 1, 128),
                                          (300, 2, 1, 1, 64), (1100, 1, 1, 2, 128)])
def test_attention_fwd_bwd(s, b, ng, qpg, d, causal):
    torch.manual_seed(0)
    q = torch.randn(s, b, ng, qpg, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(s, b, ng, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(s, b, ng, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = attention(q, k, v, causal=causal)
    torch.cuda.synchronize()
    _lib.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref_attention(qr, kr, vr, causal, 1.0 / math.sqrt(d))
    assert _rel(out, ref) < 2e-2
    do = torch.randn_like(ref)
    out.backward(do.to(out.dtype))
    ref.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(q.grad, qr.grad) < 3e-2
    assert _rel(k.grad, kr.grad) < 3e-2
    assert _rel(v.grad, vr.grad) < 3e-2


def test_attention_rectangular_causal():
    """sq < sk: the last query row sees the last key (decode / chunked prefill shape)."""
    torch.manual_seed(1)
    sq, sk, d = 128, 320, 128
    q = torch.randn(sq, 1, 2, 1, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sk, 1, 2, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sk, 1, 2, d, device="cuda", dtype=torch.bfloat16)
    out = attention(q, k, v, causal=True)
    ref = _ref_attention(q.float(), k.float(), v.float(), True, 1.0 / math.sqrt(d))
    assert _rel(out, ref) < 2e-2


def test_attention_rectangular_ragged_backward():
    """sq < sk with neither a multiple of a tile, forward and backward, causal and full."""
    torch.manual_seed(3)
    sq, sk, d = 300, 812, 128
    for causal in (True, False):
        q = torch.randn(sq, 1, 2, 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(sk, 1, 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn(sk, 1, 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        out = attention(q, k, v, causal=causal)
        qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
        ref = _ref_attention(qr, kr, vr, causal, 1.0 / math.sqrt(d))
        assert _rel(out, ref) < 2e-2
        do = torch.randn_like(ref)
        out.backward(do.to(out.dtype))
        ref.backward(do)
        torch.cuda.synchronize()
        _lib.check_status()
        for a, r in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
            assert _rel(a, r) < 3e-2


def test_attention_full_more_queries_than_keys():
    """Not causal, sq > sk: the shape of a ring-attention step that holds half of a peer's keys."""
    torch.manual_seed(5)
    sq, sk, d = 512, 256, 128
    q = torch.randn(sq, 1, 2, 1, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(sk, 1, 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(sk, 1, 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = attention(q, k, v, causal=False)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref_attention(qr, kr, vr, False, 1.0 / math.sqrt(d))
    assert _rel(out, ref) < 2e-2
    do = torch.randn_like(ref)
    out.backward(do.to(out.dtype))
    ref.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    for a, r in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert _rel(a, r) < 3e-2


@pytest.mark.parametrize("s,qpg,d,window", [(1100, 1, 128, 100), (1100, 2, 128, 128), (640, 1, 128, 300), (1024, 1, 64, 255),
                                            (512, 1, 128, 0), (700, 1, 128, 5000)])
def test_attention_sliding_window(s, qpg, d, window):
    """Causal sliding window (a query sees itself and ``window`` keys before it), forward and backward."""
    torch.manual_seed(6)
    q = torch.randn(s, 1, 2, qpg, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(s, 1, 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(s, 1, 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = attention(q, k, v, causal=True, window=window)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref_attention(qr, kr, vr, True, 1.0 / math.sqrt(d), window=window)
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(out, ref) < 2e-2
    do = torch.randn_like(ref)
    out.backward(do.to(out.dtype))
    ref.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    for a, r in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        # with window 0 every query sees one key and dq, dk are exactly zero in the reference: absolute bound then
        assert (a.float() - r).norm().item() < 3e-2 * max(r.norm().item(), 1.0)


def test_attention_large_scores_rescale():
    """Scores that grow along the keys force the running maximum up by more than the lazy-rescale threshold."""
    torch.manual_seed(4)
    s, d = 1024, 128
    q = torch.randn(s, 1, 1, 1, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(s, 1, 1, d, device="cuda", dtype=torch.bfloat16) * torch.linspace(0.2, 6.0, s, device="cuda").view(s, 1, 1, 1).to(torch.bfloat16)
    v = torch.randn(s, 1, 1, d, device="cuda", dtype=torch.bfloat16)
    for causal in (True, False):
        out = attention(q, k, v, causal=causal)
        ref = _ref_attention(q.float(), k.float(), v.float(), causal, 1.0 / math.sqrt(d))
        torch.cuda.synchronize()
        _lib.check_status()
        assert _rel(out, ref) < 2e-2


def test_attention_kernel_variants_in_a_child_process():
    """The kernels that pass P / dS through shared memory (``MLB_ATTN_FWD2=0 MLB_ATTN_TS=0``) stay correct."""
    import os
    import subprocess
    import sys
    code = (
        "import math, torch\n"
        "from megatron_lm_b200.ops import _lib\n"
        "from megatron_lm_b200.ops.attention import _ref_attention, attention\n"
        "torch.manual_seed(0)\n"
        "for s, qpg, d, causal in ((384, 2, 64, True), (1100, 1, 128, True), (200, 1, 128, False)):\n"
        "    q = torch.randn(s, 1, 2, qpg, d, device='cuda', dtype=torch.bfloat16, requires_grad=True)\n"
        "    k = torch.randn(s, 1, 2, d, device='cuda', dtype=torch.bfloat16, requires_grad=True)\n"
        "    v = torch.randn(s, 1, 2, d, device='cuda', dtype=torch.bfloat16, requires_grad=True)\n"
        "    out = attention(q, k, v, causal=causal)\n"
        "    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))\n"
        "    ref = _ref_attention(qr, kr, vr, causal, 1.0 / math.sqrt(d))\n"
        "    do = torch.randn_like(ref)\n"
        "    out.backward(do.to(out.dtype)); ref.backward(do)\n"
        "    torch.cuda.synchronize(); _lib.check_status()\n"
        "    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()\n"
        "    assert rel(out, ref) < 2e-2 and rel(q.grad, qr.grad) < 3e-2\n"
        "    assert rel(k.grad, kr.grad) < 3e-2 and rel(v.grad, vr.grad) < 3e-2\n"
        "print('ok')\n")
    env = dict(os.environ, MLB_ATTN_FWD2="0", MLB_ATTN_TS="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr


def test_fused_qkv_attention_in_place_views():
    torch.manual_seed(2)
    s, b, ng, qpg, d = 256, 2, 2, 2, 128
    qkv = torch.randn(s, b, ng, qpg + 2, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = fused_qkv_attention(qkv, causal=True)
    ref_in = qkv.detach().float().requires_grad_()
    ref = fused_qkv_attention(ref_in.cpu().requires_grad_(), causal=True) if False else None
    r = qkv.detach().float().requires_grad_()
    o = _ref_attention(r[:, :, :, :qpg], r[:, :, :, qpg], r[:, :, :, qpg + 1], True, 1.0 / math.sqrt(d))
    o = o.reshape(s, b, ng * qpg * d)
    assert _rel(out, o) < 2e-2
    do = torch.randn_like(o)
    out.backward(do.to(out.dtype))
    o.backward(do)
    assert _rel(qkv.grad, r.grad) < 3e-2
    # run-twice bitwise reproducibility (no atomics anywhere in the backward)
    qkv2 = qkv.detach().clone().requires_grad_()
    fused_qkv_attention(qkv2, causal=True).backward(do.to(out.dtype))
    assert torch.equal(qkv2.grad, qkv.grad)
    _lib.check_status()
