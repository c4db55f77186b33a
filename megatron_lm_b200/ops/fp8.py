"""FP8 training ops: quantisation (per-tensor current scaling, MXFP8 blocks) and the FP8 GEMM.

The tensor-core GEMM takes 8-bit operands K-major only, so every quantised tensor can carry its
transpose, produced in the same pass: forward multiplies X_q W_q^T, the data gradient dY_q (W_q^T)^T and
the weight gradient (dY_q^T)(X_q^T)^T, accumulated in fp32 straight into ``main_grad``.  Scales stay on the
device from amax to epilogue - no host synchronisation.  Recipe parity: "tensorwise" of the reference
(megatron/core/fp8_utils.py:459-485, Float8CurrentScaling), formats ``e4m3`` and ``hybrid`` (e5m2 for
gradients).  CPU tensors run an emulation through torch's float8 dtypes (also the test oracle).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib
from .grad import deliver, has_main_grad, notify_ready

_lib.register_signatures({
    "mlb_amax": "iplpp",
    "mlb_fp8_cast_transpose": "ipppppiiip",
    "mlb_mxfp8_quantize": "ipppiiip",
    "mlb_gemm_fp8": "iiplplpliipppiiipp",
    "mlb_mxfp8_quantize_dual": "ippppp" "iiip",
    "mlb_mx_sf_bytes": "ll",
    "mlb_gemm_mx": "iiplpplppliipiiipp",
})

_TORCH_FP8 = {0: torch.float8_e4m3fn, 1: torch.float8_e5m2}
_FMAX = {0: 448.0, 1: 57344.0}


@dataclass
class Fp8Tensor:
    data: torch.Tensor                 # uint8 [rows, cols]
    data_t: Optional[torch.Tensor]     # uint8 [cols, rows] or None
    scale_inv: torch.Tensor            # fp32 [1]: value = data * scale_inv
    fmt: int                           # 0 e4m3, 1 e5m2

    def dequantize(self) -> torch.Tensor:
        return self.data.view(_TORCH_FP8[self.fmt]).float() * self.scale_inv


def quantize(x: torch.Tensor, fmt: int = 0, transpose: bool = True) -> Fp8Tensor:
    """Per-tensor scaling with the scale taken from this tensor's own amax."""
    x2 = x.reshape(-1, x.shape[-1])
    rows, cols = x2.shape
    if not x2.is_cuda:
        a = x2.float().abs().max()
        scale = torch.where((a > 0) & torch.isfinite(a), _FMAX[fmt] / a, torch.ones_like(a))
        q = (x2.float() * scale).clamp(-_FMAX[fmt], _FMAX[fmt]).to(_TORCH_FP8[fmt]).view(torch.uint8)
        return Fp8Tensor(q, q.t().contiguous() if transpose else None, (1.0 / scale).reshape(1), fmt)
    x2 = x2.contiguous()
    L = _lib.lib()
    amax = torch.zeros(1, dtype=torch.float32, device=x.device)
    _lib.check(L.mlb_amax(_lib.dt(x2), x2.data_ptr(), x2.numel(), amax.data_ptr(), _lib.stream()), "amax")
    q = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    qt = torch.empty(cols, rows, dtype=torch.uint8, device=x.device) if transpose else None
    sinv = torch.empty(1, dtype=torch.float32, device=x.device)
    _lib.check(L.mlb_fp8_cast_transpose(_lib.dt(x2), x2.data_ptr(), amax.data_ptr(), q.data_ptr(), _lib.ptr(qt),
                                        sinv.data_ptr(), rows, cols, fmt, _lib.stream()), "fp8 cast")
    return Fp8Tensor(q, qt, sinv, fmt)


def gemm_fp8(a: torch.Tensor, a_fmt: int, a_sinv: torch.Tensor, b: torch.Tensor, b_fmt: int, b_sinv: torch.Tensor,
             out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, accumulate: bool = False,
             bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K], b [N, K] uint8 -> (a b^T) * a_sinv * b_sinv (+ bias) as [M, N]."""
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if not a.is_cuda:
        r = (a.view(_TORCH_FP8[a_fmt]).float() @ b.view(_TORCH_FP8[b_fmt]).float().t()) * (a_sinv * b_sinv)
        if bias is not None:
            r = r + bias.float()
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out
    mode = 0 if out.dtype in (torch.bfloat16, torch.float16) else (2 if accumulate else 1)
    if accumulate and mode == 0:
        raise ValueError("accumulation needs an fp32 output")
    lp = 1 if (out.dtype == torch.bfloat16 or bias is None or bias.dtype == torch.bfloat16) else 0
    if out.dtype == torch.float16:
        lp = 0
    st = _lib.status_word()
    _lib.check(_lib.lib().mlb_gemm_fp8(a_fmt, b_fmt, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(),
                                       out.stride(0), mode, lp, _lib.ptr(bias), a_sinv.data_ptr(), b_sinv.data_ptr(),
                                       M, N, K, st.data_ptr(), _lib.stream()), "gemm_fp8")
    return out


class _Fp8LinearFn(torch.autograd.Function):
    """y = x W^T (+ bias) with e4m3 operands; gradients quantised to ``grad_fmt`` (e5m2 for "hybrid")."""

    @staticmethod
    def forward(ctx, x, weight, bias, grad_fmt):
        x2 = x.reshape(-1, x.shape[-1])
        xq = quantize(x2, 0, transpose=weight.requires_grad)
        wq = quantize(weight, 0, transpose=x.requires_grad)
        y = gemm_fp8(xq.data, 0, xq.scale_inv, wq.data, 0, wq.scale_inv, out_dtype=x.dtype,
                     bias=None if bias is None else bias.to(x.dtype))
        ctx.save_for_backward(xq.data_t if xq.data_t is not None else xq.data, xq.scale_inv,
                              wq.data_t if wq.data_t is not None else wq.data, wq.scale_inv)
        ctx.weight, ctx.bias, ctx.grad_fmt, ctx.x_shape, ctx.x_dtype = weight, bias, grad_fmt, x.shape, x.dtype
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        xq_t, x_sinv, wq_t, w_sinv = ctx.saved_tensors
        weight, bias = ctx.weight, ctx.bias
        dy2 = dy.reshape(-1, dy.shape[-1])
        dq = quantize(dy2, ctx.grad_fmt, transpose=weight.requires_grad)
        dx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dx [M, K] = dy [M, N] (W^T [K, N])^T
            dx = gemm_fp8(dq.data, ctx.grad_fmt, dq.scale_inv, wq_t, 0, w_sinv, out_dtype=ctx.x_dtype).view(ctx.x_shape)
        if weight.requires_grad:
            # dW [N, K] = dy^T [N, M] (x^T [K, M])^T
            if has_main_grad(weight) and weight.main_grad.dtype == torch.float32:
                gemm_fp8(dq.data_t, ctx.grad_fmt, dq.scale_inv, xq_t, 0, x_sinv, out=weight.main_grad, accumulate=True)
                notify_ready(weight)
            else:
                g = gemm_fp8(dq.data_t, ctx.grad_fmt, dq.scale_inv, xq_t, 0, x_sinv, out_dtype=torch.float32)
                gw = deliver(weight, g)
        if bias is not None and bias.requires_grad:
            gb = deliver(bias, dy2.float().sum(dim=0))
        return dx, gw, gb, None


def linear_fp8(x, weight, bias=None, fp8_format: str = "hybrid"):
    """Drop-in linear with FP8 GEMMs.  Token count and both feature sizes must be multiples of 16."""
    return _Fp8LinearFn.apply(x, weight, bias, 1 if fp8_format == "hybrid" else 0)


# ----------------------------------------------------------------------------- MXFP8
def mxfp8_quantize(x: torch.Tensor, along_rows: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Blocks of 32 elements (along the last dim, or down the rows) share an E8M0 scale byte.
    Returns (e4m3 bytes with x's 2-d shape, scale bytes [rows, cols/32] or [rows/32, cols])."""
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    rows, cols = x2.shape
    if not x2.is_cuda:
        xf = x2.float()
        blk = xf.view(rows, cols // 32, 32) if along_rows else xf.view(rows // 32, 32, cols).transpose(1, 2)
        amax = blk.abs().amax(dim=-1)
        e = torch.where(amax > 0, torch.ceil(torch.log2(amax / 448.0)), torch.full_like(amax, -127.0)).clamp(-127, 127)
        q = (blk * torch.exp2(-e).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
        q = q.view(rows, cols) if along_rows else q.transpose(1, 2).reshape(rows, cols)
        return q.contiguous(), (e + 127).to(torch.uint8)
    q = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    sc = torch.empty((rows, cols // 32) if along_rows else (rows // 32, cols), dtype=torch.uint8, device=x.device)
    _lib.check(_lib.lib().mlb_mxfp8_quantize(_lib.dt(x2), x2.data_ptr(), q.data_ptr(), sc.data_ptr(), rows, cols,
                                             int(along_rows), _lib.stream()), "mxfp8 quantize")
    return q, sc


def mxfp8_dequantize(q: torch.Tensor, scales: torch.Tensor, along_rows: bool = True) -> torch.Tensor:
    rows, cols = q.shape
    v = q.view(torch.float8_e4m3fn).float()
    s = torch.exp2(scales.float() - 127.0)
    if along_rows:
        return (v.view(rows, cols // 32, 32) * s.unsqueeze(-1)).view(rows, cols)
    return (v.view(rows // 32, 32, cols) * s.unsqueeze(1)).view(rows, cols)


# ----------------------------------------------------------------------------- MXFP8 training GEMMs
def mx_sf_bytes(rows: int, k: int) -> int:
    """Size of the scale buffer of a quantised [rows, k] operand: atoms of 128 rows x 128 K elements, 512 B each."""
    return ((rows + 127) // 128) * ((k + 127) // 128) * 512


def mx_sf_index(rows: int, k: int, device="cpu") -> torch.Tensor:
    """[rows, k/32] int64: byte position of each (row, K block) scale in the atom layout the block-scaled GEMM
    copies to tensor memory (``csrc/gemm_mx.cu``)."""
    r = torch.arange(rows, device=device).unsqueeze(1)
    kb = torch.arange(k // 32, device=device).unsqueeze(0)
    kb4 = (k + 127) // 128
    return ((r // 128) * kb4 + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4


@dataclass
class MxTensor:
    """MXFP8 operand: ``data`` uint8 [rows, k] (K-major), ``sf`` uint8 scale bytes in the atom layout."""
    data: torch.Tensor
    sf: torch.Tensor
    fmt: int

    def dequantize(self) -> torch.Tensor:
        rows, k = self.data.shape
        e = self.sf.to("cpu")[mx_sf_index(rows, k)].float() - 127.0
        v = self.data.to("cpu").view(_TORCH_FP8[self.fmt]).float().view(rows, k // 32, 32)
        return (v * torch.exp2(e).unsqueeze(-1)).view(rows, k).to(self.data.device)


def mxfp8_quantize_dual(x: torch.Tensor, fmt: int = 0, rowwise: bool = True, colwise: bool = True
                        ) -> Tuple[Optional[MxTensor], Optional[MxTensor]]:
    """One pass over ``x`` [rows, cols] -> (row-wise copy [rows, cols] scaled along cols, column-wise copy
    transposed to [cols, rows] and scaled along rows).  The first feeds a GEMM that reduces over ``cols``, the
    second one that reduces over ``rows`` (reference: the two usages of an MXFP8 tensor,
    megatron/core/fp8_utils.py:459-485)."""
    x2 = x.reshape(-1, x.shape[-1])
    rows, cols = x2.shape
    if (rowwise and cols % 32) or (colwise and rows % 32) or cols % 8:
        raise ValueError("MXFP8 blocks of 32 need the scaled dimension to be a multiple of 32 (and rows of whole "
                         "16-byte pieces)")
    dev = x.device
    if not x2.is_cuda:
        def one(m):      # m [R, K] float -> MxTensor, scaled along K
            R, K = m.shape
            blk = m.view(R, K // 32, 32)
            amax = blk.abs().amax(dim=-1)
            e = torch.where(amax > 0, torch.ceil(torch.log2(amax / _FMAX[fmt])),
                            torch.full_like(amax, -127.0)).clamp(-127, 127)
            q = (blk * torch.exp2(-e).unsqueeze(-1)).clamp(-_FMAX[fmt], _FMAX[fmt]).to(_TORCH_FP8[fmt]).view(torch.uint8)
            sf = torch.zeros(mx_sf_bytes(R, K), dtype=torch.uint8)
            sf[mx_sf_index(R, K).reshape(-1)] = (e + 127).to(torch.uint8).reshape(-1)
            return MxTensor(q.view(R, K).contiguous(), sf, fmt)
        xf = x2.float()
        return (one(xf) if rowwise else None), (one(xf.t().contiguous()) if colwise else None)
    x2 = x2.contiguous()
    qr = sr = qc = sc = None
    if rowwise:
        qr = torch.empty(rows, cols, dtype=torch.uint8, device=dev)
        sr = torch.zeros(mx_sf_bytes(rows, cols), dtype=torch.uint8, device=dev)
    if colwise:
        qc = torch.empty(cols, rows, dtype=torch.uint8, device=dev)
        sc = torch.zeros(mx_sf_bytes(cols, rows), dtype=torch.uint8, device=dev)
    _lib.check(_lib.lib().mlb_mxfp8_quantize_dual(_lib.dt(x2), x2.data_ptr(), _lib.ptr(qr), _lib.ptr(sr), _lib.ptr(qc),
                                                  _lib.ptr(sc), rows, cols, fmt, _lib.stream()), "mxfp8 quantize")
    return (MxTensor(qr, sr, fmt) if rowwise else None), (MxTensor(qc, sc, fmt) if colwise else None)


def gemm_mx(a: MxTensor, b: MxTensor, out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
            accumulate: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M, K], b [N, K] MXFP8 -> a b^T (+ bias) as [M, N] on the block-scaled tensor-core path."""
    M, K = a.data.shape
    N = b.data.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.data.device)
    if not a.data.is_cuda:
        r = a.dequantize() @ b.dequantize().t()
        if bias is not None:
            r = r + bias.float()
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out
    mode = 0 if out.dtype in (torch.bfloat16, torch.float16) else (2 if accumulate else 1)
    if accumulate and mode == 0:
        raise ValueError("accumulation needs an fp32 output")
    lp = 0 if (out.dtype == torch.float16 or (bias is not None and bias.dtype == torch.float16)) else 1
    st = _lib.status_word()
    _lib.check(_lib.lib().mlb_gemm_mx(a.fmt, b.fmt, a.data.data_ptr(), a.data.stride(0), a.sf.data_ptr(),
                                      b.data.data_ptr(), b.data.stride(0), b.sf.data_ptr(), out.data_ptr(),
                                      out.stride(0), mode, lp, _lib.ptr(bias), M, N, K, st.data_ptr(), _lib.stream()),
               "gemm_mx")
    return out


# Quantised copies of a weight are reused by every microbatch of a step: the optimizer announces new weights by
# advancing this counter (the bf16 weights are rewritten through raw pointers, which tensor version counters
# do not see).
_WEIGHT_EPOCH = [0]


def weights_updated() -> None:
    _WEIGHT_EPOCH[0] += 1


def _quantized_weight(weight: torch.Tensor, need_col: bool):
    c = getattr(weight, "_mx_cache", None)
    key = (_WEIGHT_EPOCH[0], weight.data_ptr(), weight._version)
    if c is not None and c[0] == key and (c[2] is not None or not need_col):
        return c[1], c[2]
    wr, wc = mxfp8_quantize_dual(weight.detach(), 0, colwise=need_col)
    weight._mx_cache = (key, wr, wc)
    return wr, wc


class _MxLinearFn(torch.autograd.Function):
    """y = x W^T (+ bias) with MXFP8 operands (1 x 32 blocks, power-of-two scales): activations and weights e4m3,
    gradients ``grad_fmt``.  Every tensor is quantised once into the two copies its GEMMs need."""

    @staticmethod
    def forward(ctx, x, weight, bias, grad_fmt):
        x2 = x.reshape(-1, x.shape[-1])
        xr, xc = mxfp8_quantize_dual(x2, 0, colwise=weight.requires_grad)
        wr, wc = _quantized_weight(weight, x.requires_grad)
        y = gemm_mx(xr, wr, out_dtype=x.dtype, bias=None if bias is None else bias.to(x.dtype))
        ctx.xc, ctx.wc = xc, wc
        ctx.weight, ctx.bias, ctx.grad_fmt, ctx.x_shape, ctx.x_dtype = weight, bias, grad_fmt, x.shape, x.dtype
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        weight, bias = ctx.weight, ctx.bias
        dy2 = dy.reshape(-1, dy.shape[-1])
        dr, dc = mxfp8_quantize_dual(dy2, ctx.grad_fmt, rowwise=ctx.needs_input_grad[0], colwise=weight.requires_grad)
        dx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dx [T, K] = dy [T, N] (W^T [K, N])^T: reduction over N
            dx = gemm_mx(dr, ctx.wc, out_dtype=ctx.x_dtype).view(ctx.x_shape)
        if weight.requires_grad:
            # dW [N, K] = dy^T [N, T] (x^T [K, T])^T: reduction over tokens
            if has_main_grad(weight) and weight.main_grad.dtype == torch.float32:
                gemm_mx(dc, ctx.xc, out=weight.main_grad, accumulate=True)
                notify_ready(weight)
            else:
                gw = deliver(weight, gemm_mx(dc, ctx.xc, out_dtype=torch.float32))
        if bias is not None and bias.requires_grad:
            gb = deliver(bias, dy2.float().sum(dim=0))
        ctx.xc = ctx.wc = None
        return dx, gw, gb, None


def linear_mxfp8(x, weight, bias=None, fp8_format: str = "hybrid"):
    """Drop-in linear with block-scaled FP8 GEMMs.  Token count and both feature sizes must be multiples of 32."""
    return _MxLinearFn.apply(x, weight, bias, 1 if fp8_format == "hybrid" else 0)


# ----------------------------------------------------------------------------- delayed scaling
class DelayedScalingState:
    """Scale taken from the amax history of *previous* steps (no extra pass over the tensor before the cast):
    ``fp8_amax_history_len`` past maxima, reduced with ``max`` or ``most_recent``; scale = fp8_max / amax / 2^margin
    (reference: the "delayed" recipe configured at megatron/core/fp8_utils.py:459-470 and its ``TEDelayedScaling``
    wrapper, extensions/transformer_engine.py:1462)."""

    def __init__(self, fmt: int = 0, history_len: int = 1, algo: str = "most_recent", margin: int = 0, device="cpu"):
        self.fmt, self.algo, self.margin = fmt, algo, margin
        self.history = torch.zeros(history_len, dtype=torch.float32, device=device)
        self.scale = torch.ones(1, dtype=torch.float32, device=device)

    def _update(self, amax: torch.Tensor) -> None:
        self.history = torch.roll(self.history, 1)
        self.history[0] = amax
        ref = self.history.max() if self.algo == "max" else self.history[0]
        s = _FMAX[self.fmt] / ref / (2.0 ** self.margin)
        self.scale = torch.where((ref > 0) & torch.isfinite(s), s, self.scale).reshape(1)

    def quantize(self, x: torch.Tensor, transpose: bool = False) -> Fp8Tensor:
        """Cast with the current scale, then fold this tensor's amax into the history for the next call."""
        x2 = x.reshape(-1, x.shape[-1])
        scale = self.scale.to(x2.device)
        q = (x2.float() * scale).clamp(-_FMAX[self.fmt], _FMAX[self.fmt]).to(_TORCH_FP8[self.fmt]).view(torch.uint8)
        out = Fp8Tensor(q, q.t().contiguous() if transpose else None, (1.0 / scale).reshape(1), self.fmt)
        self.history = self.history.to(x2.device)
        self._update(x2.detach().float().abs().max())
        return out


def quantize_param_shard(master_shard: torch.Tensor, fmt: int = 0, amax_group=None) -> Fp8Tensor:
    """FP8 copy of an fp32 master-weight shard for the parameter all-gather (``--fp8-param-gather``): the amax is
    reduced over ``amax_group`` first so that every shard of one tensor uses the same scale
    (reference: fp8_utils.py:394)."""
    import torch.distributed as dist
    a = master_shard.detach().float().abs().max().reshape(1)
    if amax_group is not None and dist.is_initialized():
        dist.all_reduce(a, op=dist.ReduceOp.MAX, group=amax_group)
    scale = torch.where(a > 0, _FMAX[fmt] / a, torch.ones_like(a))
    flat = master_shard.reshape(1, -1)
    q = (flat.float() * scale).clamp(-_FMAX[fmt], _FMAX[fmt]).to(_TORCH_FP8[fmt]).view(torch.uint8)
    return Fp8Tensor(q, None, 1.0 / scale, fmt)
