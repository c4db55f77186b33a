"""Flash attention over strided q/k/v views (no split or transpose copies).

Tensors are in the reference's [s, b, heads, head_dim] convention
(megatron/core/transformer/attention.py:537-781).  ``q`` has ``ng * qpg`` heads
organised as ``ng`` KV groups of ``qpg`` query heads; ``k``/``v`` have ``ng``
heads.  Any strides are allowed on the s, b and head dims as long as head_dim is
contiguous, so the three tensors may be views of one fused QKV projection
output [s, b, ng, qpg + 2, hn] - the TMA descriptors address them in place, and
the backward writes dq/dk/dv into one fused gradient buffer of the same layout.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib

_lib.register_signatures({
    # fmt, q,k,v,o,lse, sq,sk,b,ng,qpg,hn, q strides(s,b,g,j) k(s,b,g) v(s,b,g) o(s,b,g,j), scale, causal, status, stream
    "mlb_attn_fwd": "ippppp" "iiiiii" "llll" "lll" "lll" "llll" "fii" "pp",
    # fmt, q,k,v,o,do,lse,delta, dq,dk,dv, sizes, strides q,k,v,o,do(s,b,g,j), dq(s,b,g,j), dk, dv, scale, causal, status, stream
    "mlb_attn_bwd": "ipppppppppp" "iiiiii" "llll" "lll" "lll" "llll" "llll" "llll" "lll" "lll" "fii" "pp",
})


def _ref_attention(q, k, v, causal: bool, scale: float, q_offset: int = 0, window: Optional[int] = None):
    # q [sq, b, ng, qpg, d]; k, v [sk, b, ng, d]
    sq, b, ng, qpg, d = q.shape
    sk = k.shape[0]
    qf = q.float().permute(1, 2, 3, 0, 4)                      # b ng qpg sq d
    kf = k.float().permute(1, 2, 0, 3).unsqueeze(2)            # b ng 1 sk d
    vf = v.float().permute(1, 2, 0, 3).unsqueeze(2)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale         # b ng qpg sq sk
    if causal:
        i = torch.arange(sq, device=q.device).unsqueeze(1) + q_offset + (sk - sq if q_offset == 0 else 0)
        j = torch.arange(sk, device=q.device).unsqueeze(0)
        s = s.masked_fill(j > i, float("-inf"))
        if window is not None:
            s = s.masked_fill(j < i - window, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vf)                                    # b ng qpg sq d
    return o.permute(3, 0, 1, 2, 4).reshape(sq, b, ng * qpg, d).to(q.dtype)


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, window=-1):
        sq, b, ng, qpg, d = q.shape
        sk = k.shape[0]
        assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
        o = torch.empty(sq, b, ng, qpg, d, dtype=q.dtype, device=q.device)
        lse = torch.empty(b, ng, qpg, sq, dtype=torch.float32, device=q.device)
        st = _lib.status_word()
        qs, ks, vs, os_ = q.stride(), k.stride(), v.stride(), o.stride()
        _lib.check(_lib.lib().mlb_attn_fwd(
            1 if q.dtype == torch.bfloat16 else 0, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
            lse.data_ptr(), sq, sk, b, ng, qpg, d, qs[0], qs[1], qs[2], qs[3], ks[0], ks[1], ks[2],
            vs[0], vs[1], vs[2], os_[0], os_[1], os_[2], os_[3], float(scale), int(causal), int(window), st.data_ptr(),
            _lib.stream()), "attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cfg = (causal, scale, window)
        return o.view(sq, b, ng * qpg, d)

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale, window = ctx.cfg
        sq, b, ng, qpg, d = q.shape
        sk = k.shape[0]
        do = do.reshape(sq, b, ng, qpg, d)
        if do.stride(-1) != 1:
            do = do.contiguous()
        dq = torch.empty(sq, b, ng, qpg, d, dtype=q.dtype, device=q.device)
        dk = torch.empty(sk, b, ng, d, dtype=q.dtype, device=q.device)
        dv = torch.empty(sk, b, ng, d, dtype=q.dtype, device=q.device)
        delta = torch.empty(b, ng, qpg, sq, dtype=torch.float32, device=q.device)
        st = _lib.status_word()
        qs, ks, vs, os_, dos = q.stride(), k.stride(), v.stride(), o.stride(), do.stride()
        dqs, dks, dvs = dq.stride(), dk.stride(), dv.stride()
        _lib.check(_lib.lib().mlb_attn_bwd(
            1 if q.dtype == torch.bfloat16 else 0, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
            do.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            sq, sk, b, ng, qpg, d, qs[0], qs[1], qs[2], qs[3], ks[0], ks[1], ks[2], vs[0], vs[1], vs[2],
            os_[0], os_[1], os_[2], os_[3], dos[0], dos[1], dos[2], dos[3], dqs[0], dqs[1], dqs[2], dqs[3],
            dks[0], dks[1], dks[2], dvs[0], dvs[1], dvs[2], float(scale), int(causal), int(window), st.data_ptr(),
            _lib.stream()), "attn_bwd")
        return dq, dk, dv, None, None, None


class _FusedQKVAttnFn(torch.autograd.Function):
    """Attention on a fused QKV activation [s, b, ng, qpg + 2, hn]; the gradient comes back as
    one tensor of the same layout, ready to be the QKV GEMM's output gradient."""

    @staticmethod
    def forward(ctx, qkv, causal, scale, cos, sin, interleaved, window=-1):
        s, b, ng, tot, d = qkv.shape
        qpg = tot - 2
        if cos is not None:
            # Rotate q and k inside the projection output itself.  Its producer keeps no
            # reference to it for backward, and the rotation is undone on the gradient below.
            from .core import _rope_launch
            qk = qkv[:, :, :, :qpg + 1]
            _rope_launch(qk, qk, cos, sin, interleaved, 1.0)
        ctx.rope = (cos, sin, interleaved)
        q, k, v = qkv[:, :, :, :qpg], qkv[:, :, :, qpg], qkv[:, :, :, qpg + 1]
        o = torch.empty(s, b, ng, qpg, d, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(b, ng, qpg, s, dtype=torch.float32, device=qkv.device)
        st = _lib.status_word()
        qs, ks, vs, os_ = q.stride(), k.stride(), v.stride(), o.stride()
        _lib.check(_lib.lib().mlb_attn_fwd(
            1 if qkv.dtype == torch.bfloat16 else 0, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
            lse.data_ptr(), s, s, b, ng, qpg, d, qs[0], qs[1], qs[2], qs[3], ks[0], ks[1], ks[2],
            vs[0], vs[1], vs[2], os_[0], os_[1], os_[2], os_[3], float(scale), int(causal), int(window), st.data_ptr(),
            _lib.stream()), "attn_fwd")
        ctx.save_for_backward(qkv, o, lse)
        ctx.cfg = (causal, scale, window)
        return o.view(s, b, ng * qpg * d)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        causal, scale, window = ctx.cfg
        s, b, ng, tot, d = qkv.shape
        qpg = tot - 2
        q, k, v = qkv[:, :, :, :qpg], qkv[:, :, :, qpg], qkv[:, :, :, qpg + 1]
        do = do.reshape(s, b, ng, qpg, d)
        if do.stride(-1) != 1:
            do = do.contiguous()
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :, :qpg], dqkv[:, :, :, qpg], dqkv[:, :, :, qpg + 1]
        delta = torch.empty(b, ng, qpg, s, dtype=torch.float32, device=qkv.device)
        st = _lib.status_word()
        qs, ks, vs, os_, dos = q.stride(), k.stride(), v.stride(), o.stride(), do.stride()
        dqs, dks, dvs = dq.stride(), dk.stride(), dv.stride()
        _lib.check(_lib.lib().mlb_attn_bwd(
            1 if qkv.dtype == torch.bfloat16 else 0, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
            do.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            s, s, b, ng, qpg, d, qs[0], qs[1], qs[2], qs[3], ks[0], ks[1], ks[2], vs[0], vs[1], vs[2],
            os_[0], os_[1], os_[2], os_[3], dos[0], dos[1], dos[2], dos[3], dqs[0], dqs[1], dqs[2], dqs[3],
            dks[0], dks[1], dks[2], dvs[0], dvs[1], dvs[2], float(scale), int(causal), int(window), st.data_ptr(),
            _lib.stream()), "attn_bwd")
        cos, sin, interleaved = ctx.rope
        if cos is not None:
            from .core import _rope_launch
            dqk = dqkv[:, :, :, :qpg + 1]
            _rope_launch(dqk, dqk, cos, sin, interleaved, -1.0)       # inverse rotation of dq, dk
        return dqkv, None, None, None, None, None, None


# ----------------------------------------------------------------------------- raw forward / backward
def attention_fwd_raw(q, k, v, causal: bool, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(o [sq, b, ng, qpg, d], lse [b, ng, qpg, sq] natural log) without autograd - the building block
    of ring attention, which merges partial results by their log-sum-exp."""
    sq, b, ng, qpg, d = q.shape
    sk = k.shape[0]
    if not q.is_cuda:
        qf = q.float().permute(1, 2, 3, 0, 4)
        kf = k.float().permute(1, 2, 0, 3).unsqueeze(2)
        vf = v.float().permute(1, 2, 0, 3).unsqueeze(2)
        s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
        if causal:
            i = torch.arange(sq).unsqueeze(1) + (sk - sq)
            s = s.masked_fill(torch.arange(sk).unsqueeze(0) > i, float("-inf"))
        lse = torch.logsumexp(s, dim=-1)
        o = torch.matmul(torch.exp(s - lse.unsqueeze(-1)), vf)
        return o.permute(3, 0, 1, 2, 4).to(q.dtype).contiguous(), lse
    o = torch.empty(sq, b, ng, qpg, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(b, ng, qpg, sq, dtype=torch.float32, device=q.device)
    st = _lib.status_word()
    qs, ks, vs, os_ = q.stride(), k.stride(), v.stride(), o.stride()
    _lib.check(_lib.lib().mlb_attn_fwd(
        1 if q.dtype == torch.bfloat16 else 0, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
        sq, sk, b, ng, qpg, d, qs[0], qs[1], qs[2], qs[3], ks[0], ks[1], ks[2], vs[0], vs[1], vs[2],
        os_[0], os_[1], os_[2], os_[3], float(scale), int(causal), -1, st.data_ptr(), _lib.stream()), "attn_fwd")
    return o, lse


def attention_bwd_raw(q, k, v, o, do, lse, causal: bool, scale: float):
    """(dq, dk, dv) of one attention block given the *final* output ``o`` and log-sum-exp ``lse`` of
    the rows (which may come from a merge over several blocks)."""
    sq, b, ng, qpg, d = q.shape
    sk = k.shape[0]
    if not q.is_cuda:
        qf = q.float().permute(1, 2, 3, 0, 4)
        kf = k.float().permute(1, 2, 0, 3).unsqueeze(2)
        vf = v.float().permute(1, 2, 0, 3).unsqueeze(2)
        dof = do.float().permute(1, 2, 3, 0, 4)
        of = o.float().permute(1, 2, 3, 0, 4)
        s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
        if causal:
            i = torch.arange(sq).unsqueeze(1) + (sk - sq)
            s = s.masked_fill(torch.arange(sk).unsqueeze(0) > i, float("-inf"))
        p = torch.exp(s - lse.unsqueeze(-1))
        delta = (dof * of).sum(-1, keepdim=True)
        dv = torch.matmul(p.transpose(-1, -2), dof).sum(2)                 # sum over q heads of the group
        dp = torch.matmul(dof, vf.transpose(-1, -2))
        ds = p * (dp - delta) * scale
        dq = torch.matmul(ds, kf)
        dk = torch.matmul(ds.transpose(-1, -2), qf).sum(2)
        return (dq.permute(3, 0, 1, 2, 4).to(q.dtype).contiguous(), dk.permute(2, 0, 1, 3).to(q.dtype).contiguous(),
                dv.permute(2, 0, 1, 3).to(q.dtype).contiguous())
    do = do if do.stride(-1) == 1 else do.contiguous()
    dq = torch.empty(sq, b, ng, qpg, d, dtype=q.dtype, device=q.device)
    dk = torch.empty(sk, b, ng, d, dtype=q.dtype, device=q.device)
    dv = torch.empty(sk, b, ng, d, dtype=q.dtype, device=q.device)
    delta = torch.empty(b, ng, qpg, sq, dtype=torch.float32, device=q.device)
    st = _lib.status_word()
    qs, ks, vs, os_, dos = q.stride(), k.stride(), v.stride(), o.stride(), do.stride()
    dqs, dks, dvs = dq.stride(), dk.stride(), dv.stride()
    _lib.check(_lib.lib().mlb_attn_bwd(
        1 if q.dtype == torch.bfloat16 else 0, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
        lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), sq, sk, b, ng, qpg, d,
        qs[0], qs[1], qs[2], qs[3], ks[0], ks[1], ks[2], vs[0], vs[1], vs[2], os_[0], os_[1], os_[2], os_[3],
        dos[0], dos[1], dos[2], dos[3], dqs[0], dqs[1], dqs[2], dqs[3], dks[0], dks[1], dks[2], dvs[0], dvs[1], dvs[2],
        float(scale), int(causal), -1, st.data_ptr(), _lib.stream()), "attn_bwd")
    return dq, dk, dv


def attention(q, k, v, causal: bool = True, scale: Optional[float] = None, window: Optional[int] = None):
    """q [sq, b, ng, qpg, d], k/v [sk, b, ng, d] -> [sq, b, ng*qpg, d].  With ``causal`` the last
    query row attends to the last key (sq <= sk); ``window`` (causal only) limits a query to itself and the
    ``window`` keys before it (reference: the ``window_size=(left, 0)`` the attention back end receives,
    megatron/core/extensions/transformer_engine.py:786-800)."""
    d = q.shape[-1]
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    if window is not None and not causal:
        raise ValueError("the sliding window is the causal one")
    if not q.is_cuda:
        return _ref_attention(q, k, v, causal, scale, window=window)
    return _FlashAttnFn.apply(q, k, v, causal, scale, -1 if window is None else int(window))


def fused_qkv_attention(qkv5, causal: bool = True, scale: Optional[float] = None, rope=None,
                        rotary_interleaved: bool = False, window: Optional[int] = None):
    """Self-attention straight from the fused projection [s, b, ng, qpg + 2, hn] -> [s, b, np*hn].
    ``rope=(cos, sin)`` (fp32 [s, rot/2]) rotates q and k first; on CUDA this happens in place in
    ``qkv5``, which must therefore not be read again by the caller.  ``window``: causal sliding window."""
    if window is not None and not causal:
        raise ValueError("the sliding window is the causal one")
    s, b, ng, tot, d = qkv5.shape
    scale = (1.0 / math.sqrt(d)) if scale is None else scale
    cos, sin = rope if rope is not None else (None, None)
    if not qkv5.is_cuda:
        qpg = tot - 2
        if cos is not None:
            from .core import apply_rope_qkv_
            qkv5 = apply_rope_qkv_(qkv5, cos, sin, rotary_interleaved)
        o = _ref_attention(qkv5[:, :, :, :qpg], qkv5[:, :, :, qpg], qkv5[:, :, :, qpg + 1], causal, scale, window=window)
        return o.reshape(s, b, ng * qpg * d)
    return _FusedQKVAttnFn.apply(qkv5, causal, scale, cos, sin, rotary_interleaved, -1 if window is None else int(window))
