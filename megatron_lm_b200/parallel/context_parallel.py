"""Context parallelism: every activation is sharded along the sequence over the CP group; only
attention communicates.  The sequence is cut into 2*cp chunks and rank r holds chunks r and
2cp-1-r, which balances causal work (reference: megatron/core/utils.py:1833,
models/common/embeddings/rope_utils.py:48-70).  The reference delegates the attention itself to
Transformer Engine (extensions/transformer_engine.py:705-876, ``cp_comm_type``); here the three
schemes are written on top of this library's flash-attention kernels:

* ``p2p``        ring attention: K/V blocks travel round the ring (async send/recv on the CP group)
                 while the current block is attended; partial outputs are merged by log-sum-exp;
                 backward sends dK/dV round the ring the same way.  With the zig-zag layout a step
                 is one of three dense shapes: own block -> causal; block of an earlier rank -> all
                 queries x its first chunk; block of a later rank -> second query chunk x all keys.
* ``all_gather`` gather K/V once (cheap for GQA), two causal calls per rank with sq < sk.
* ``a2a``        Ulysses: all-to-all to [full sequence, heads / cp], local attention, all-to-all back.
* ``a2a+p2p``    hierarchical: Ulysses inside the inner sub-group (consecutive ranks, e.g. one NVLink island),
                 ring attention between the sub-groups.  After the inner all-to-all a rank holds, for its share
                 of the heads, the early chunks of its whole sub-group and their mirror late chunks - again a
                 zig-zag layout, of the sub-groups - so the ring step logic is reused unchanged
                 (reference: megatron/core/parallel_state.py:305-364 builds the groups,
                 extensions/transformer_engine.py:876-930 passes them to the attention).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from . import state
from .mappings import all_to_all
from ..ops.attention import attention, attention_bwd_raw, attention_fwd_raw


def zigzag_indices(seq_len: int, cp: int, rank: int, device=None) -> torch.Tensor:
    """Global positions of this rank's tokens: chunks ``rank`` and ``2cp-1-rank`` of 2cp."""
    c = seq_len // (2 * cp)
    a = torch.arange(rank * c, (rank + 1) * c, device=device)
    b = torch.arange((2 * cp - 1 - rank) * c, (2 * cp - rank) * c, device=device)
    return torch.cat((a, b))


def natural_order_permutation(seq_len: int, cp: int, device=None) -> torch.Tensor:
    """Index that sorts the rank-concatenated zig-zag sequence back into natural order."""
    order = torch.cat([zigzag_indices(seq_len, cp, r, device) for r in range(cp)])
    return torch.argsort(order)


def _merge(o, lse, o_i, lse_i):
    """Fold a partial (o_i, lse_i) into the running (o, lse); o: [s,b,ng,qpg,d], lse: [b,ng,qpg,s]."""
    if o is None:
        return o_i.float(), lse_i
    new = torch.logaddexp(lse, lse_i)
    w_old = torch.exp(lse - new).permute(3, 0, 1, 2).unsqueeze(-1)
    w_new = torch.exp(lse_i - new).permute(3, 0, 1, 2).unsqueeze(-1)
    return o * w_old + o_i.float() * w_new, new


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, scale, causal):
        cp, r = dist.get_world_size(group), dist.get_rank(group)
        nxt = dist.get_global_rank(group, (r + 1) % cp)
        prv = dist.get_global_rank(group, (r - 1) % cp)
        s = q.shape[0]
        half = s // 2
        kv = torch.stack((k, v)).contiguous()
        o = lse = None
        blocks = []
        for step in range(cp):
            reqs, kv_next = [], None
            if step + 1 < cp:
                kv_next = torch.empty_like(kv)
                reqs = dist.batch_isend_irecv([dist.P2POp(dist.isend, kv, nxt, group),
                                               dist.P2POp(dist.irecv, kv_next, prv, group)])
            src = (r - step) % cp
            kb, vb = kv[0], kv[1]
            if not causal or src == r:
                o_i, lse_i = attention_fwd_raw(q, kb, vb, causal, scale)
                o, lse = _merge(o, lse, o_i, lse_i)
            elif src < r:
                o_i, lse_i = attention_fwd_raw(q, kb[:half], vb[:half], False, scale)
                o, lse = _merge(o, lse, o_i, lse_i)
            else:
                o_i, lse_i = attention_fwd_raw(q[half:], kb, vb, False, scale)
                o2, l2 = _merge(o[half:], lse[..., half:], o_i, lse_i)
                o = torch.cat((o[:half], o2))
                lse = torch.cat((lse[..., :half], l2), dim=-1)
            for w in reqs:
                w.wait()
            if kv_next is not None:
                kv = kv_next
        out = o.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse.contiguous())
        ctx.cfg = (group, scale, causal)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        group, scale, causal = ctx.cfg
        cp, r = dist.get_world_size(group), dist.get_rank(group)
        nxt = dist.get_global_rank(group, (r + 1) % cp)
        prv = dist.get_global_rank(group, (r - 1) % cp)
        s = q.shape[0]
        half = s // 2
        do = do.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        kv = torch.stack((k, v)).contiguous()
        dkv = torch.zeros_like(kv, dtype=torch.float32)        # travels with its K/V block
        for step in range(cp):
            src = (r - step) % cp
            kb, vb = kv[0], kv[1]
            if not causal or src == r:
                dq_i, dk_i, dv_i = attention_bwd_raw(q, kb, vb, o, do, lse, causal, scale)
                dq += dq_i.float()
                dkv[0] += dk_i.float()
                dkv[1] += dv_i.float()
            elif src < r:
                dq_i, dk_i, dv_i = attention_bwd_raw(q, kb[:half], vb[:half], o, do, lse, False, scale)
                dq += dq_i.float()
                dkv[0, :half] += dk_i.float()
                dkv[1, :half] += dv_i.float()
            else:
                dq_i, dk_i, dv_i = attention_bwd_raw(q[half:], kb, vb, o[half:], do[half:],
                                                     lse[..., half:].contiguous(), False, scale)
                dq[half:] += dq_i.float()
                dkv[0] += dk_i.float()
                dkv[1] += dv_i.float()
            # pass the block and its gradient accumulator on; after cp steps both are home again
            kv_next, dkv_next = torch.empty_like(kv), torch.empty_like(dkv)
            ops = [dist.P2POp(dist.isend, dkv, nxt, group), dist.P2POp(dist.irecv, dkv_next, prv, group)]
            if step + 1 < cp:
                ops += [dist.P2POp(dist.isend, kv, nxt, group), dist.P2POp(dist.irecv, kv_next, prv, group)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()
            dkv = dkv_next
            if step + 1 < cp:
                kv = kv_next
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None


def ring_attention(q, k, v, group=None, scale: Optional[float] = None, causal: bool = True):
    """q [s_local, b, ng, qpg, d], k/v [s_local, b, ng, d] in zig-zag layout -> [s_local, b, ng*qpg, d]."""
    group = group if group is not None else state.get_context_parallel_group()
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if group is None or dist.get_world_size(group) == 1:
        return attention(q, k, v, causal, scale)
    o = _RingAttention.apply(q, k, v, group, scale, causal)
    return o.reshape(o.shape[0], o.shape[1], -1, o.shape[-1])


class _GatherSeq(torch.autograd.Function):
    """all-gather along dim 0 whose backward is a reduce-scatter (sum of every rank's gradient)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        out = torch.empty((x.shape[0] * n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        out = torch.empty((g.shape[0] // n,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def allgather_attention(q, k, v, group=None, scale: Optional[float] = None, causal: bool = True):
    group = group if group is not None else state.get_context_parallel_group()
    if group is None or dist.get_world_size(group) == 1:
        return attention(q, k, v, causal, scale)
    cp, r = dist.get_world_size(group), dist.get_rank(group)
    s_local = q.shape[0]
    S = s_local * cp
    c = s_local // 2
    perm = natural_order_permutation(S, cp, q.device)
    kf = _GatherSeq.apply(k, group).index_select(0, perm)
    vf = _GatherSeq.apply(v, group).index_select(0, perm)
    if not causal:
        return attention(q, kf, vf, False, scale)
    e0, e1 = (r + 1) * c, (2 * cp - r) * c               # one past the last key each query chunk may see
    o0 = attention(q[:c], kf[:e0], vf[:e0], True, scale)
    o1 = attention(q[c:], kf[:e1], vf[:e1], True, scale)
    return torch.cat((o0, o1), dim=0)


def ulysses_attention(q, k, v, group=None, scale: Optional[float] = None, causal: bool = True):
    """Trade sequence sharding for head sharding around a local full-sequence attention."""
    group = group if group is not None else state.get_context_parallel_group()
    if group is None or dist.get_world_size(group) == 1:
        return attention(q, k, v, causal, scale)
    cp = dist.get_world_size(group)
    s_local, b, ng, qpg, d = q.shape
    if ng % cp != 0:
        raise ValueError("the a2a scheme needs the number of KV groups to be divisible by the CP size")
    S = s_local * cp
    perm = natural_order_permutation(S, cp, q.device)
    inv = torch.argsort(perm)

    def seq_to_heads(t):          # [s_local, b, ng, ...] -> [S (natural order), b, ng/cp, ...]
        rest = t.shape[3:]
        x = t.reshape(s_local, b, cp, ng // cp, *rest).permute(2, 0, 1, 3, *range(4, 4 + len(rest))).contiguous()
        x = all_to_all(group, x.reshape(cp * s_local, b, ng // cp, *rest))
        return x.index_select(0, perm)

    def heads_to_seq(t):          # [S natural, b, ng/cp, qpg, d] -> [s_local, b, ng, qpg, d]
        x = all_to_all(group, t.index_select(0, inv).contiguous())
        x = x.reshape(cp, s_local, b, ng // cp, qpg, d).permute(1, 2, 0, 3, 4, 5)
        return x.reshape(s_local, b, ng, qpg, d)

    o = attention(seq_to_heads(q), seq_to_heads(k), seq_to_heads(v), causal, scale)
    o = o.reshape(S, b, ng // cp, qpg, d)
    out = heads_to_seq(o)
    return out.reshape(s_local, b, ng * qpg, d)


def hierarchical_attention(q, k, v, inner_group, outer_group, scale: Optional[float] = None, causal: bool = True):
    """``a2a+p2p``: q [s_local, b, ng, qpg, d], k/v [s_local, b, ng, d] in the zig-zag layout of the whole
    context-parallel group (size = inner x outer, inner ranks consecutive) -> [s_local, b, ng*qpg, d]."""
    A = dist.get_world_size(inner_group)
    if A == 1:
        return ring_attention(q, k, v, outer_group, scale, causal)
    s_local, b, ng, qpg, d = q.shape
    if ng % A != 0:
        raise ValueError("a2a+p2p needs the number of KV groups to be divisible by the inner (a2a) group size")
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    c = s_local // 2
    # gathered order is (source rank j, [early chunk, late chunk]); wanted: early chunks by rank, then late chunks by
    # falling rank - natural order inside both halves, which is what the ring's zig-zag steps assume
    pos = torch.arange(A * s_local, device=q.device).view(A, 2, c)
    order = torch.cat((pos[:, 0].reshape(-1), pos[:, 1].flip(0).reshape(-1)))
    inv = torch.argsort(order)

    def seq_to_heads(t):          # [s_local, b, ng, ...] -> [A * s_local, b, ng / A, ...]
        rest = t.shape[3:]
        x = t.reshape(s_local, b, A, ng // A, *rest).permute(2, 0, 1, 3, *range(4, 4 + len(rest))).contiguous()
        x = all_to_all(inner_group, x.reshape(A * s_local, b, ng // A, *rest))
        return x.index_select(0, order)

    def heads_to_seq(t):          # [A * s_local, b, ng / A, qpg, d] -> [s_local, b, ng, qpg, d]
        x = all_to_all(inner_group, t.index_select(0, inv).contiguous())
        x = x.reshape(A, s_local, b, ng // A, qpg, d).permute(1, 2, 0, 3, 4, 5)
        return x.reshape(s_local, b, ng, qpg, d)

    o = ring_attention(seq_to_heads(q), seq_to_heads(k), seq_to_heads(v), outer_group, scale, causal)
    out = heads_to_seq(o.reshape(A * s_local, b, ng // A, qpg, d))
    return out.reshape(s_local, b, ng * qpg, d)


def context_parallel_attention(q, k, v, comm_type: str = "p2p", group=None, scale=None, causal=True):
    if comm_type == "p2p":
        return ring_attention(q, k, v, group, scale, causal)
    if comm_type == "all_gather":
        return allgather_attention(q, k, v, group, scale, causal)
    if comm_type == "a2a":
        return ulysses_attention(q, k, v, group, scale, causal)
    if comm_type == "a2a+p2p":
        groups = state.get_hierarchical_context_parallel_groups()
        if len(groups) < 2:
            return ring_attention(q, k, v, group, scale, causal)
        # level 0 is the innermost (fastest varying) sub-group: all-to-all there, ring across
        return hierarchical_attention(q, k, v, groups[0], groups[1], scale, causal)
    raise ValueError(f"unknown cp_comm_type {comm_type}")
