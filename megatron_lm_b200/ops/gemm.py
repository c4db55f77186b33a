"""GEMM and the linear layer's three products on the tcgen05 kernel.

``gemm`` exposes the kernel's operand-layout freedom (each operand K-major or
MN-major), which is what lets forward, data-gradient and weight-gradient products
all read the tensors autograd already holds, with no transposed copies.  The
weight gradient is accumulated in fp32 straight into ``weight.main_grad`` when
the parameter has one (reference behaviour: ``gradient_accumulation_fusion``,
megatron/core/tensor_parallel/layers.py:553-598).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .core import column_sum
from .grad import deliver, has_main_grad, notify_ready

OUT_LP, OUT_F32, OUT_F32_ACC = 0, 1, 2


def _as2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 2 and t.stride(1) == 1:
        return t
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.stride(1) == 1 else t2.contiguous()


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, accumulate: bool = False,
         bias: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    """D[M,N] (=|+=) op(a) @ op(b)^T-style product.

    a: [M,K] (``a_mn=False``) or stored [K,M] (``a_mn=True``);
    b: [N,K] (``b_mn=False``) or stored [K,N] (``b_mn=True``).
    ``out`` may be a bf16/fp16 or fp32 2-d tensor with unit inner stride; ``accumulate``
    needs an fp32 ``out``."""
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    if K != Kb:
        raise ValueError(f"reduction dims differ: {K} vs {Kb}")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    if not a.is_cuda:
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        r = A.float() @ B.float()
        if bias is not None:
            r = r + bias.float()
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out
    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("the tcgen05 GEMM takes bf16 or fp16 operands of one dtype")
    if out.dtype == torch.float32:
        mode = OUT_F32_ACC if accumulate else OUT_F32
    else:
        if accumulate or out.dtype != a.dtype:
            raise TypeError("accumulate needs an fp32 output; low-precision output must match the input dtype")
        mode = OUT_LP
    assert out.stride(1) == 1 and out.shape[0] == M and out.shape[1] == N
    if bias is not None:
        bias = bias.to(a.dtype).contiguous()
    st = _lib.status_word()
    stream = _lib.stream()
    args = (1 if a.dtype == torch.bfloat16 else 0, a.data_ptr(), a.stride(0), int(a_mn),
            b.data_ptr(), b.stride(0), int(b_mn), out.data_ptr(), out.stride(0), mode,
            _lib.ptr(bias), M, N, K, max_ctas, st.data_ptr(), stream)
    if _PAIR and N >= 256 and M >= 256 and (out.stride(0) * out.element_size()) % 16 == 0 and out.data_ptr() % 16 == 0:
        # CTA-pair kernel: 256 x 256 tiles over two SMs
        _lib.check(_lib.lib().mlb_gemm_pair(*args, _sched_words(stream) if _DYNAMIC else None), "gemm")
    else:
        _lib.check(_lib.lib().mlb_gemm(*args), "gemm")
    return out


import os as _os

_PAIR = _os.environ.get("MLB_GEMM_PAIR", "1") == "1"      # set MLB_GEMM_PAIR=0 for the single-CTA kernel
# Dynamic tile schedule of the CTA-pair kernel (tiles drawn from a device counter by whichever blocks are running).
# With the static schedule a persistent grid needs a second wave whenever another stream's long-running kernel
# (pipeline send / receive, gradient reduction) holds a few SMs: the blocks that found no SM still own their share
# of the tiles.  The training set-up turns this on when such kernels exist; MLB_GEMM_DYNAMIC=0/1 forces it.
_DYNAMIC = _os.environ.get("MLB_GEMM_DYNAMIC", "0") == "1"
_sched = {}


def set_dynamic_schedule(on: bool) -> None:
    global _DYNAMIC
    env = _os.environ.get("MLB_GEMM_DYNAMIC")
    _DYNAMIC = (env == "1") if env in ("0", "1") else bool(on)


def _sched_words(stream: int) -> Optional[int]:
    """Two zeroed words per (device, stream): launches on one stream are ordered, so they can share them.  None (static
    schedule) for a stream first seen while it is being captured into a graph: nothing may be allocated then."""
    key = (_lib.device_index(), stream)
    t = _sched.get(key)
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        with torch.cuda.stream(torch.cuda.default_stream()):
            t = torch.zeros(2, dtype=torch.int32, device="cuda")
        torch.cuda.default_stream().synchronize()
        _sched[key] = t
    return t.data_ptr()


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, wgrad_deferred):
        x2 = _as2d(x)
        y = gemm(x2, weight, bias=bias)
        ctx.save_for_backward(x2, weight)
        ctx.bias = bias
        ctx.x_shape = x.shape
        ctx.deferred = wgrad_deferred
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = _as2d(dy)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        gw = None
        if weight.requires_grad:
            gw = weight_grad(weight, dy2, x2)
        gb = None
        if ctx.bias is not None and ctx.bias.requires_grad:
            gb = deliver(ctx.bias, column_sum(dy2))
        return dx, gw, gb, None


def weight_grad(weight: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor) -> Optional[torch.Tensor]:
    """dW = dy^T x, accumulated into ``weight.main_grad`` when present."""
    if has_main_grad(weight) and weight.main_grad.dtype == torch.float32:
        gemm(dy2, x2, a_mn=True, b_mn=True, out=weight.main_grad.view(weight.shape), accumulate=True)
        notify_ready(weight)
        return None
    g = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32)
    return deliver(weight, g)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ weight^T + bias with weight [out, in]."""
    if not x.is_cuda:
        return torch.nn.functional.linear(x, weight, bias)
    return _LinearFn.apply(x, weight, bias, False)
