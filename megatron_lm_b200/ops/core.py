"""Fused ops of the transformer layer outside GEMM and attention.

Every op has two bodies: plain differentiable PyTorch on CPU tensors (this is
also the fp32 oracle the GPU tests compare with) and a ``torch.autograd.Function``
over the sm_100a kernels of ``csrc/`` on CUDA tensors.  On CUDA there is no other
implementation to fall back to.
"""
from __future__ import annotations

import ctypes

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from .grad import deliver, has_main_grad, notify_ready
from ..utils.memory import workspace


def _rows(x: torch.Tensor) -> int:
    return x.numel() // x.shape[-1]


# --------------------------------------------------------------------------- norms
def _norm_ref(x, weight, bias, eps, rms, zero_centered):
    w = weight.float() + 1.0 if zero_centered else weight.float()
    xf = x.float()
    if rms:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w
    else:
        mu = xf.mean(-1, keepdim=True)
        var = (xf - mu).pow(2).mean(-1, keepdim=True)
        y = (xf - mu) * torch.rsqrt(var + eps) * w
        if bias is not None:
            y = y + bias.float()
    return y.to(x.dtype)


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms, zero_centered):
        xc = x.contiguous()
        h = xc.shape[-1]
        rows = _rows(xc)
        y = torch.empty_like(xc)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        mean = rstd if rms else torch.empty(rows, dtype=torch.float32, device=x.device)
        wc = weight.to(xc.dtype) if weight.dtype != xc.dtype else weight
        bc = None if bias is None else (bias.to(xc.dtype) if bias.dtype != xc.dtype else bias)
        _lib.check(_lib.lib().mlb_norm_fwd(_lib.dt(xc), int(rms), xc.data_ptr(), wc.data_ptr(), _lib.ptr(bc),
                                           y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, h, float(eps),
                                           int(zero_centered), _lib.stream()), "norm_fwd")
        ctx.save_for_backward(xc, wc, mean, rstd)
        ctx.cfg = (rms, zero_centered, weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, wc, mean, rstd = ctx.saved_tensors
        rms, zc, weight, bias = ctx.cfg
        dy = dy.contiguous()
        h = xc.shape[-1]
        rows = _rows(xc)
        L = _lib.lib()
        grid = L.mlb_norm_bwd_grid(rows)
        ws = workspace((grid, 2, h), torch.float32, "norm_bwd", xc.device)
        dx = torch.empty_like(xc)
        direct = has_main_grad(weight) and weight.main_grad.dtype == torch.float32 and \
            (bias is None or (has_main_grad(bias) and bias.main_grad.dtype == torch.float32))
        if direct:
            dg = weight.main_grad
            db = bias.main_grad if bias is not None else None
        else:
            dg = torch.empty(h, dtype=torch.float32, device=xc.device)
            db = torch.empty(h, dtype=torch.float32, device=xc.device) if (bias is not None and not rms) else None
        _lib.check(L.mlb_norm_bwd(_lib.dt(xc), int(rms), dy.data_ptr(), xc.data_ptr(), wc.data_ptr(),
                                  mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dg.data_ptr(), _lib.ptr(db),
                                  ws.data_ptr(), rows, h, int(zc), int(direct), _lib.stream()), "norm_bwd")
        if direct:
            notify_ready(weight)
            if bias is not None:
                notify_ready(bias)
            return dx, None, None, None, None, None
        gw = deliver(weight, dg) if weight.requires_grad else None
        gb = deliver(bias, db) if (bias is not None and db is not None and bias.requires_grad) else None
        return dx, gw, gb, None, None, None


def rmsnorm(x, weight, eps: float = 1e-5, zero_centered_gamma: bool = False):
    if not x.is_cuda:
        return _norm_ref(x, weight, None, eps, True, zero_centered_gamma)
    return _NormFn.apply(x, weight, None, eps, True, zero_centered_gamma)


def layernorm(x, weight, bias=None, eps: float = 1e-5, zero_centered_gamma: bool = False):
    if not x.is_cuda:
        return _norm_ref(x, weight, bias, eps, False, zero_centered_gamma)
    return _NormFn.apply(x, weight, bias, eps, False, zero_centered_gamma)


# --------------------------------------------------------------------------- activations
def _swiglu_ref(x):
    a, b = x.float().chunk(2, dim=-1)
    return (F.silu(a) * b).to(x.dtype)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        f = xc.shape[-1] // 2
        out = torch.empty(*xc.shape[:-1], f, dtype=xc.dtype, device=xc.device)
        _lib.check(_lib.lib().mlb_swiglu_fwd(_lib.dt(xc), xc.data_ptr(), out.data_ptr(), _rows(xc), f, _lib.stream()),
                   "swiglu_fwd")
        ctx.save_for_backward(xc)
        return out

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dy = dy.contiguous()
        f = xc.shape[-1] // 2
        dx = torch.empty_like(xc)
        _lib.check(_lib.lib().mlb_swiglu_bwd(_lib.dt(xc), dy.data_ptr(), xc.data_ptr(), dx.data_ptr(), _rows(xc), f,
                                             _lib.stream()), "swiglu_bwd")
        return dx


def swiglu(x):
    """silu(x[..., :f]) * x[..., f:] (reference: fusions/fused_bias_swiglu.py:16)."""
    return _SwiGLUFn.apply(x) if x.is_cuda else _swiglu_ref(x)


def _gelu_ref(x, bias):
    v = x.float() if bias is None else x.float() + bias.float()
    return F.gelu(v, approximate="tanh").to(x.dtype)


def column_sum(x2d: torch.Tensor) -> torch.Tensor:
    """fp32 sum over rows of a [rows, cols] tensor (bias gradients)."""
    if not x2d.is_cuda:
        return x2d.float().sum(0)
    L = _lib.lib()
    rows, cols = x2d.shape
    parts = L.mlb_colsum_parts(rows)
    ws = workspace((parts, cols), torch.float32, "colsum", x2d.device)
    out = torch.empty(cols, dtype=torch.float32, device=x2d.device)
    _lib.check(L.mlb_colsum(_lib.dt(x2d), x2d.data_ptr(), out.data_ptr(), ws.data_ptr(), rows, cols, 0,
                            _lib.stream()), "colsum")
    return out


class _BiasGeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        xc = x.contiguous()
        f = xc.shape[-1]
        bc = None if bias is None else bias.to(xc.dtype)
        out = torch.empty_like(xc)
        _lib.check(_lib.lib().mlb_bias_gelu_fwd(_lib.dt(xc), xc.data_ptr(), _lib.ptr(bc), out.data_ptr(), _rows(xc),
                                                f, _lib.stream()), "bias_gelu_fwd")
        ctx.save_for_backward(xc, bc)
        ctx.bias = bias
        return out

    @staticmethod
    def backward(ctx, dy):
        xc, bc = ctx.saved_tensors
        dy = dy.contiguous()
        f = xc.shape[-1]
        dx = torch.empty_like(xc)
        _lib.check(_lib.lib().mlb_bias_gelu_bwd(_lib.dt(xc), dy.data_ptr(), xc.data_ptr(), _lib.ptr(bc),
                                                dx.data_ptr(), _rows(xc), f, _lib.stream()), "bias_gelu_bwd")
        gb = None
        if ctx.bias is not None and ctx.bias.requires_grad:
            gb = deliver(ctx.bias, column_sum(dx.view(-1, f)))
        return dx, gb


def bias_gelu(x, bias=None):
    """tanh-form GeLU of x + bias (reference: fusions/fused_bias_gelu.py:17)."""
    return _BiasGeluFn.apply(x, bias) if x.is_cuda else _gelu_ref(x, bias)


# --------------------------------------------------------------------------- RoPE
def rope_tables(seq_len: int, rot_dim: int, base: float = 10000.0, device=None, positions=None,
                scaling_factor: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables [seq, rot_dim/2]; ``inv_freq = base^(-2i/rot_dim)``
    (reference: models/common/embeddings/rotary_pos_embedding.py:36)."""
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    pos = torch.arange(seq_len, dtype=torch.float32, device=device) if positions is None else positions.float()
    if scaling_factor:
        pos = pos / scaling_factor
    ang = torch.outer(pos, inv)
    return ang.cos().contiguous(), ang.sin().contiguous()


def _rope_ref(t, cos, sin, interleaved, sign=1.0):
    # t [s, b, n, hn]; cos/sin [s, rot/2]
    rot = cos.shape[-1] * 2
    tr, tp = t[..., :rot].float(), t[..., rot:]
    c = cos[:, None, None, :]
    s = sin[:, None, None, :] * sign
    if interleaved:
        x0, x1 = tr[..., 0::2], tr[..., 1::2]
        o = torch.stack((x0 * c - x1 * s, x1 * c + x0 * s), dim=-1).flatten(-2)
    else:
        x0, x1 = tr[..., : rot // 2], tr[..., rot // 2:]
        o = torch.cat((x0 * c - x1 * s, x1 * c + x0 * s), dim=-1)
    return torch.cat((o.to(t.dtype), tp), dim=-1)


def _rope_launch(src, dst, cos, sin, interleaved, sign):
    # src/dst: 5-d views [s, b, n_outer, n_inner, hn] with hn contiguous
    s, b, no, ni, hn = src.shape
    assert src.stride(-1) == 1 and dst.stride(-1) == 1
    ss, ds = src.stride(), dst.stride()
    _lib.check(_lib.lib().mlb_rope(_lib.dt(src), src.data_ptr(), dst.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                   s, b, no, ni, hn, cos.shape[-1] * 2, int(interleaved), float(sign),
                                   ss[0], ss[1], ss[2], ss[3], ds[0], ds[1], ds[2], ds[3], _lib.stream()), "rope")


class _RopeFn(torch.autograd.Function):
    """Out-of-place RoPE on a [s, b, n, hn] tensor (any s/b/n strides)."""

    @staticmethod
    def forward(ctx, t, cos, sin, interleaved):
        out = torch.empty(t.shape, dtype=t.dtype, device=t.device)
        _rope_launch(t.unsqueeze(2), out.unsqueeze(2), cos, sin, interleaved, 1.0)
        ctx.save_for_backward(cos, sin)
        ctx.interleaved = interleaved
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        if dy.stride(-1) != 1:
            dy = dy.contiguous()
        dx = torch.empty(dy.shape, dtype=dy.dtype, device=dy.device)
        _rope_launch(dy.unsqueeze(2), dx.unsqueeze(2), cos, sin, ctx.interleaved, -1.0)
        return dx, None, None, None


def apply_rope(t, cos, sin, interleaved: bool = False):
    """Rotate the first ``2*cos.shape[-1]`` channels of each head of ``t`` [s, b, n, hn]."""
    if not t.is_cuda:
        return _rope_ref(t, cos, sin, interleaved)
    return _RopeFn.apply(t, cos, sin, interleaved)


class _RopeQKVInplaceFn(torch.autograd.Function):
    """RoPE applied in place to the query and key heads of a fused QKV tensor
    [s, b, ng, (q_per_group + 2), hn]; value heads are untouched.  The rotation is
    orthogonal, so backward is the inverse rotation of the incoming gradient and
    needs no saved activation."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, interleaved):
        view = qkv[:, :, :, :-1, :]
        _rope_launch(view, view, cos, sin, interleaved, 1.0)
        ctx.mark_dirty(qkv)
        ctx.save_for_backward(cos, sin)
        ctx.interleaved = interleaved
        return qkv

    @staticmethod
    def backward(ctx, d):
        cos, sin = ctx.saved_tensors
        d = d.clone(memory_format=torch.contiguous_format)   # the incoming gradient may have other readers
        view = d[:, :, :, :-1, :]
        _rope_launch(view, view, cos, sin, ctx.interleaved, -1.0)
        return d, None, None, None


def apply_rope_qkv_(qkv5, cos, sin, interleaved: bool = False):
    """In-place RoPE on q and k inside a fused QKV activation (see class doc)."""
    if not qkv5.is_cuda:
        qk = _rope_ref(qkv5[:, :, :, :-1, :].flatten(2, 3), cos, sin, interleaved).view_as(qkv5[:, :, :, :-1, :])
        return torch.cat((qk, qkv5[:, :, :, -1:, :]), dim=3)
    return _RopeQKVInplaceFn.apply(qkv5, cos, sin, interleaved)


# --------------------------------------------------------------------------- bias + dropout + add
class _BDAFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p, seed, offset):
        xc, rc = x.contiguous(), residual.contiguous()
        h = xc.shape[-1]
        bc = None if bias is None else bias.to(xc.dtype)
        out = torch.empty_like(xc)
        mask = torch.empty(xc.numel() // 8, dtype=torch.uint8, device=xc.device) if p > 0 else None
        _lib.check(_lib.lib().mlb_bias_dropout_add(_lib.dt(xc), xc.data_ptr(), _lib.ptr(bc), rc.data_ptr(),
                                                   out.data_ptr(), _lib.ptr(mask), _rows(xc), h, float(p),
                                                   int(seed), int(offset), _lib.stream()), "bias_dropout_add")
        ctx.p = p
        ctx.bias = bias
        if mask is not None:
            ctx.save_for_backward(mask)
        return out

    @staticmethod
    def backward(ctx, dout):
        dout = dout.contiguous()
        if ctx.p > 0:
            (mask,) = ctx.saved_tensors
            dx = torch.empty_like(dout)
            _lib.check(_lib.lib().mlb_dropout_bwd(_lib.dt(dout), dout.data_ptr(), mask.data_ptr(), dx.data_ptr(),
                                                  dout.numel(), float(ctx.p), _lib.stream()), "dropout_bwd")
        else:
            dx = dout
        gb = None
        if ctx.bias is not None and ctx.bias.requires_grad:
            gb = deliver(ctx.bias, column_sum(dx.view(-1, dx.shape[-1])))
        return dx, gb, dout, None, None, None


_bda_offset = 0


def bias_dropout_add(x, bias, residual, p: float, training: bool, seed: Optional[int] = None):
    """residual + dropout(x + bias) (reference: fusions/fused_bias_dropout.py:11-81).
    The CUDA kernel draws its mask from a counter-based hash of (seed, running offset);
    the seed comes from the active RNG tracker state so that sequence-parallel ranks differ."""
    global _bda_offset
    p = p if training else 0.0
    if not x.is_cuda:
        v = x if bias is None else x + bias
        return residual + F.dropout(v, p=p, training=p > 0)
    if p == 0.0 and bias is None:
        return residual + x
    if seed is None:
        seed = int(torch.cuda.initial_seed()) & 0x7FFFFFFFFFFFFFFF
    off = _bda_offset
    _bda_offset = (_bda_offset + x.numel()) & 0x7FFFFFFFFFFFFFFF
    return _BDAFn.apply(x, bias, residual, p, seed, off)


# --------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, weight, v0, v1):
        idx = idx.contiguous()
        h = weight.shape[1]
        out = torch.empty(*idx.shape, h, dtype=weight.dtype, device=weight.device)
        _lib.check(_lib.lib().mlb_embedding_fwd(_lib.dt(weight), idx.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                                idx.numel(), h, v0, v1, _lib.stream()), "embedding_fwd")
        ctx.save_for_backward(idx)
        ctx.w = weight
        ctx.rng = (v0, v1)
        return out

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        w = ctx.w
        dy = dy.contiguous()
        h = w.shape[1]
        direct = has_main_grad(w) and w.main_grad.dtype == torch.float32
        dw = w.main_grad if direct else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        _lib.check(_lib.lib().mlb_embedding_bwd(_lib.dt(dy), idx.data_ptr(), dy.data_ptr(), dw.data_ptr(),
                                                idx.numel(), h, ctx.rng[0], ctx.rng[1], _lib.stream()),
                   "embedding_bwd")
        if direct:
            notify_ready(w)
            return None, None, None, None
        return None, deliver(w, dw), None, None


def embedding(idx, weight, vocab_start: int = 0, vocab_end: Optional[int] = None):
    """Rows of ``weight`` for ids in [vocab_start, vocab_end); zeros elsewhere - the
    vocab-parallel shard lookup (reference: tensor_parallel/layers.py:262-295)."""
    if vocab_end is None:
        vocab_end = vocab_start + weight.shape[0]
    if not weight.is_cuda:
        mask = (idx < vocab_start) | (idx >= vocab_end)
        local = (idx - vocab_start).masked_fill(mask, 0)
        out = F.embedding(local, weight)
        return out.masked_fill(mask.unsqueeze(-1), 0.0)
    return _EmbeddingFn.apply(idx, weight, int(vocab_start), int(vocab_end))


# --------------------------------------------------------------------------- cross entropy
def _tp_reduce(t, op, group):
    if group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
        torch.distributed.all_reduce(t, op=op, group=group)
    return t


_CE_PEER = {}


class CrossEntropyPeerComm:
    """Per-row statistics table in symmetric memory for the vocab-parallel cross entropy: every rank's forward kernel
    stores its (max, sum exp, target logit, sum of logits) into all ranks' tables, a device-side barrier follows,
    and a small kernel combines the slots - no all-reduce.  Enabled with ``MLB_CE_PEER=1`` (single node)."""

    def __init__(self, group, rows: int):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.tp, self.rank, self.rows = torch.distributed.get_world_size(group), torch.distributed.get_rank(group), rows
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm_mem.empty(self.tp * rows * 4, dtype=torch.float32, device=dev)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.ptrs = (ctypes.c_void_p * self.tp)(*[int(p) for p in self.hdl.buffer_ptrs])
        self.hdl.barrier()

    @staticmethod
    def get(group, rows):
        key = (id(group), rows)
        if key not in _CE_PEER:
            _CE_PEER[key] = CrossEntropyPeerComm(group, rows)
        return _CE_PEER[key]


def _ce_peer_enabled(group, lg) -> bool:
    import os
    return os.environ.get("MLB_CE_PEER", "0") == "1" and group is not None and torch.distributed.is_initialized() \
        and 1 < torch.distributed.get_world_size(group) <= 8


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, vocab_start, vocab_total, label_smoothing, group, inplace_backward):
        v_local = logits.shape[-1]
        lg = logits.contiguous().view(-1, v_local)
        tg = target.contiguous().view(-1)
        rows = lg.shape[0]
        stats = torch.empty(4, rows, dtype=torch.float32, device=lg.device)
        if _ce_peer_enabled(group, lg):
            comm = CrossEntropyPeerComm.get(group, rows)
            L = _lib.lib()
            comm.hdl.barrier()                   # the previous call's combine has read every slot
            _lib.check(L.mlb_ce_fwd_peer(_lib.dt(lg), lg.data_ptr(), tg.data_ptr(), stats[0].data_ptr(),
                                         stats[1].data_ptr(), stats[2].data_ptr(), stats[3].data_ptr(), rows, v_local,
                                         lg.stride(0), vocab_start, comm.ptrs, comm.tp, comm.rank, comm.rows,
                                         _lib.stream()), "ce_fwd_peer")
            comm.hdl.barrier()                   # every rank's statistics have landed
            out = torch.empty(3, rows, dtype=torch.float32, device=lg.device)
            _lib.check(L.mlb_ce_combine(comm.buf.data_ptr(), comm.tp, rows, comm.rows, float(label_smoothing),
                                        vocab_total, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                        _lib.stream()), "ce_combine")
            ctx.save_for_backward(lg, tg, out[1], out[2])
            ctx.cfg = (vocab_start, vocab_total, label_smoothing, inplace_backward, logits.shape)
            return out[0].view(target.shape)
        _lib.check(_lib.lib().mlb_ce_fwd(_lib.dt(lg), lg.data_ptr(), tg.data_ptr(), stats[0].data_ptr(),
                                         stats[1].data_ptr(), stats[2].data_ptr(), stats[3].data_ptr(), rows,
                                         v_local, lg.stride(0), vocab_start, _lib.stream()), "ce_fwd")
        lmax = stats[0]
        gmax = _tp_reduce(lmax.clone(), torch.distributed.ReduceOp.MAX, group)
        # one fused reduction for (sumexp rescaled to the global max, target logit, sum of logits)
        packed = torch.stack((stats[1] * torch.exp(lmax - gmax), stats[2], stats[3]))
        packed = _tp_reduce(packed, torch.distributed.ReduceOp.SUM, group)
        gsum, tgt, sumx = packed[0], packed[1], packed[2]
        lse = torch.log(gsum) + gmax
        loss = lse - tgt
        if label_smoothing > 0:
            # (1-ls)*nll + ls * mean_over_vocab(-log p)
            smooth = lse - sumx / vocab_total
            loss = (1.0 - label_smoothing) * loss + label_smoothing * smooth
        ctx.save_for_backward(lg, tg, gmax, gsum)
        ctx.cfg = (vocab_start, vocab_total, label_smoothing, inplace_backward, logits.shape)
        return loss.view(target.shape)

    @staticmethod
    def backward(ctx, dloss):
        lg, tg, gmax, gsum = ctx.saved_tensors
        v0, vt, ls, inplace, shape = ctx.cfg
        g = dloss.contiguous().view(-1).float()
        out = lg if inplace else torch.empty_like(lg)
        _lib.check(_lib.lib().mlb_ce_bwd(_lib.dt(lg), lg.data_ptr(), tg.data_ptr(), gmax.data_ptr(), gsum.data_ptr(),
                                         g.data_ptr(), out.data_ptr(), lg.shape[0], lg.shape[1], lg.stride(0), v0,
                                         float(ls), vt, _lib.stream()), "ce_bwd")
        return out.view(shape), None, None, None, None, None, None


def _ce_ref(logits, target, vocab_start, vocab_total, label_smoothing, group):
    lf = logits.float()
    v_local = lf.shape[-1]
    lmax = lf.max(-1).values
    gmax = _tp_reduce(lmax.detach().clone(), torch.distributed.ReduceOp.MAX, group)
    shifted = lf - gmax.unsqueeze(-1)
    local = target - vocab_start
    in_range = (local >= 0) & (local < v_local)
    tgt = shifted.gather(-1, local.clamp(0, v_local - 1).unsqueeze(-1)).squeeze(-1) * in_range
    sumexp = shifted.exp().sum(-1)
    sumx = shifted.sum(-1)
    if group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
        from ..parallel.mappings import reduce_from_tensor_model_parallel_region as _ar
        tgt, sumexp, sumx = _ar(tgt, group), _ar(sumexp, group), _ar(sumx, group)
    loss = torch.log(sumexp) - tgt
    if label_smoothing > 0:
        smooth = torch.log(sumexp) - sumx / vocab_total
        loss = (1.0 - label_smoothing) * loss + label_smoothing * smooth
    return loss


def cross_entropy(logits, target, vocab_start: int = 0, vocab_total: Optional[int] = None,
                  label_smoothing: float = 0.0, group=None, inplace_backward: bool = True):
    """Per-token loss from this rank's vocab shard of the logits (fp32 result, shape of
    ``target``).  ``inplace_backward`` lets the gradient overwrite the logits buffer."""
    if vocab_total is None:
        vocab_total = logits.shape[-1]
    if not logits.is_cuda:
        return _ce_ref(logits, target, vocab_start, vocab_total, label_smoothing, group)
    return _CrossEntropyFn.apply(logits, target, int(vocab_start), int(vocab_total), float(label_smoothing), group,
                                 inplace_backward)
