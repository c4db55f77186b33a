"""Flat-buffer optimizer primitives (AdamW/SGD step, sum of squares, scale, zero count).

A *chunk table* describes a flat fp32 buffer as pieces of at most ``CHUNK``
elements, none of which crosses a parameter boundary, each tagged with its
hyper-parameter group; one kernel launch then updates the whole buffer.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from ..utils.memory import workspace

CHUNK = 16384


def build_chunk_table(segments: Sequence[Tuple[int, int, int]], device) -> Tuple[torch.Tensor, int]:
    """segments: (start, length, group) in elements of the flat buffer.  Returns the device
    table (as int32 words of {int64 start, int32 len, int32 group}) and the chunk count."""
    recs = []
    for start, length, group in segments:
        o = 0
        while o < length:
            n = min(CHUNK, length - o)
            recs.append((start + o, n, group))
            o += n
    arr = np.zeros(len(recs), dtype=np.dtype([("start", "<i8"), ("len", "<i4"), ("group", "<i4")]))
    for i, (s, n, g) in enumerate(recs):
        arr[i] = (s, n, g)
    t = torch.from_numpy(arr.view(np.int32).copy()).to(device)
    return t, len(recs)


def _farr(vals: Sequence[float]):
    return (ctypes.c_float * len(vals))(*[float(v) for v in vals])


def adam_step(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, *, table, nchunks: int,
              lrs: Sequence[float], wds: Sequence[float], beta1: float, beta2: float, eps: float, step: int,
              p_lp: Optional[torch.Tensor] = None, grad_scale: Optional[torch.Tensor] = None,
              skip: Optional[torch.Tensor] = None, segments=None, peer_lp: Optional[Sequence[int]] = None) -> None:
    """In-place AdamW (decoupled weight decay) on flat fp32 p/m/v with grads g (fp32 or bf16).
    ``grad_scale`` and ``skip`` are 1-element fp32 device tensors read by the kernel, so the
    host never waits for the clip coefficient or the overflow flag.  ``peer_lp``: device addresses (peer-mapped)
    that receive the low-precision result as well - the update then doubles as the parameter all-gather."""
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    if not p.is_cuda:
        if skip is not None and float(skip) != 0.0:
            return
        gs = 1.0 if grad_scale is None else float(grad_scale)
        for (start, length, group) in segments:
            sl = slice(start, start + length)
            gr = g[sl].float() * gs
            m[sl].mul_(beta1).add_(gr, alpha=1 - beta1)
            v[sl].mul_(beta2).addcmul_(gr, gr, value=1 - beta2)
            denom = (v[sl] / bc2).sqrt_().add_(eps)
            p[sl].mul_(1 - lrs[group] * wds[group]).addcdiv_(m[sl], denom, value=-lrs[group] / bc1)
            if p_lp is not None:
                p_lp[sl].copy_(p[sl])
        return
    if peer_lp:
        if g.dtype != torch.float32 or p_lp is None:
            raise ValueError("the peer-push update needs fp32 gradients and a low-precision parameter copy")
        arr = (ctypes.c_void_p * len(peer_lp))(*[int(a) for a in peer_lp])
        _lib.check(_lib.lib().mlb_adam_push(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), p_lp.data_ptr(), arr,
                                            len(peer_lp), table.data_ptr(), nchunks, _farr(lrs), _farr(wds), len(lrs),
                                            beta1, beta2, eps, bc1, bc2, _lib.ptr(grad_scale), _lib.ptr(skip),
                                            _lib.stream()), "adam_push")
        return
    _lib.check(_lib.lib().mlb_adam(_lib.dt(g), p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                   _lib.ptr(p_lp), table.data_ptr(), nchunks, _farr(lrs), _farr(wds), len(lrs),
                                   beta1, beta2, eps, bc1, bc2, _lib.ptr(grad_scale), _lib.ptr(skip),
                                   _lib.stream()), "adam")


def sgd_step(p, mom, g, *, table, nchunks, lrs, wds, momentum: float, first_step: bool, p_lp=None,
             grad_scale=None, skip=None, segments=None) -> None:
    if not p.is_cuda:
        if skip is not None and float(skip) != 0.0:
            return
        gs = 1.0 if grad_scale is None else float(grad_scale)
        for (start, length, group) in segments:
            sl = slice(start, start + length)
            gr = g[sl].float() * gs + wds[group] * p[sl]
            if momentum != 0.0:
                if first_step:
                    mom[sl].copy_(gr)
                else:
                    mom[sl].mul_(momentum).add_(gr)
                gr = mom[sl]
            p[sl].add_(gr, alpha=-lrs[group])
            if p_lp is not None:
                p_lp[sl].copy_(p[sl])
        return
    _lib.check(_lib.lib().mlb_sgd(_lib.dt(g), p.data_ptr(), _lib.ptr(mom), g.data_ptr(), _lib.ptr(p_lp),
                                  table.data_ptr(), nchunks, _farr(lrs), _farr(wds), len(lrs), momentum,
                                  int(first_step), _lib.ptr(grad_scale), _lib.ptr(skip), _lib.stream()), "sgd")


def grad_pull(src_addrs: Sequence[int], out: torch.Tensor, scale: float, sumsq: Optional[torch.Tensor] = None,
              accumulate: bool = True) -> None:
    """out = scale * sum of the fp32 buffers at ``src_addrs`` (this rank's and its peers' gradient slices), and
    optionally sumsq (+)= |out|^2 - the reduce-scatter of the distributed optimizer as one pull kernel."""
    L = _lib.lib()
    ws = workspace((L.mlb_sumsq_parts(),), torch.float32, "sumsq", out.device)
    arr = (ctypes.c_void_p * len(src_addrs))(*[int(a) for a in src_addrs])
    _lib.check(L.mlb_grad_pull(arr, len(src_addrs), out.data_ptr(), out.numel(), float(scale), _lib.ptr(sumsq),
                               ws.data_ptr(), int(accumulate), _lib.stream()), "grad_pull")


def grad_pull_when_ready(src_addrs: Sequence[int], out: torch.Tensor, scale: float, flags: torch.Tensor,
                         target: int, max_blocks: int = 0, workspace_tag: str = "pull-side") -> None:
    """:func:`grad_pull` behind an in-kernel wait until every word of ``flags`` (written by the peers) has reached
    ``target``.  Meant for a side stream: it gets a workspace of its own."""
    L = _lib.lib()
    ws = workspace((L.mlb_sumsq_parts(),), torch.float32, workspace_tag, out.device)
    arr = (ctypes.c_void_p * len(src_addrs))(*[int(a) for a in src_addrs])
    st = _lib.status_word()
    _lib.check(L.mlb_grad_pull_when_ready(arr, len(src_addrs), out.data_ptr(), out.numel(), float(scale), ws.data_ptr(),
                                          flags.data_ptr(), flags.numel(), int(target) & 0xFFFFFFFF, int(max_blocks),
                                          st.data_ptr(), _lib.stream()), "grad_pull")


def peer_signal(dst_addrs: Sequence[int], value: int) -> None:
    """Store ``value`` into the 32-bit word at each (peer-mapped) address, after all earlier work of the stream."""
    arr = (ctypes.c_void_p * len(dst_addrs))(*[int(a) for a in dst_addrs])
    _lib.check(_lib.lib().mlb_peer_signal(arr, len(dst_addrs), int(value) & 0xFFFFFFFF, _lib.stream()), "peer_signal")


def sum_squares(x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """fp32 1-element tensor with sum(x^2) (deterministic two-stage reduction)."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
        accumulate = False
    if not x.is_cuda:
        s = x.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s
        return out
    x = x.contiguous().view(-1)
    L = _lib.lib()
    ws = workspace((L.mlb_sumsq_parts(),), torch.float32, "sumsq", x.device)
    _lib.check(L.mlb_sumsq(_lib.dt(x), x.data_ptr(), x.numel(), out.data_ptr(), ws.data_ptr(), int(accumulate),
                           _lib.stream()), "sumsq")
    return out


def scale_(x: torch.Tensor, scale: float = 1.0, scale_tensor: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not x.is_cuda:
        x.mul_(scale if scale_tensor is None else scale * float(scale_tensor))
        return x
    assert x.is_contiguous()
    _lib.check(_lib.lib().mlb_scale(_lib.dt(x), x.data_ptr(), x.numel(), _lib.ptr(scale_tensor), float(scale),
                                    _lib.stream()), "scale")
    return x


def count_zeros(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return (x == 0).sum().to(torch.int64).view(1)
    out = torch.zeros(1, dtype=torch.int64, device=x.device)
    x = x.contiguous()
    _lib.check(_lib.lib().mlb_count_zeros(_lib.dt(x), x.data_ptr(), x.numel(), out.data_ptr(), _lib.stream()),
               "count_zeros")
    return out


def cast_copy(src: torch.Tensor, dst: torch.Tensor, scale: float = 1.0, accumulate: bool = False) -> torch.Tensor:
    """dst (=|+=) src * scale with dtype conversion (flat, 16-byte aligned buffers)."""
    if not src.is_cuda:
        if accumulate:
            dst.add_(src.to(dst.dtype) * scale)
        else:
            dst.copy_(src.to(dst.dtype) * scale)
        return dst
    assert src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel()
    _lib.check(_lib.lib().mlb_cast(_lib.dt(src), _lib.dt(dst), src.data_ptr(), dst.data_ptr(), src.numel(),
                                   float(scale), int(accumulate), _lib.stream()), "cast")
    return dst
