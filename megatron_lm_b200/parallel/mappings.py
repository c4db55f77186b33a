"""Conjugate communication pairs used by tensor / sequence / expert parallelism.

Each public function is an autograd-aware collective whose backward is its
conjugate (reference: megatron/core/tensor_parallel/mappings.py:197-538):

    copy_to_tp        identity  <-> all-reduce
    reduce_from_tp    all-reduce <-> identity
    scatter_to_tp     split(last) <-> gather(last)
    gather_from_tp    gather(last) <-> split(last)
    scatter_to_sp     split(first) <-> gather(first)
    gather_from_sp    gather(first) <-> reduce-scatter(first) (or split)
    reduce_scatter_to_sp  reduce-scatter(first) <-> gather(first)
    all_to_all        all-to-all(splits) <-> all-to-all(reversed splits)

All take an explicit process group (default: the TP group) and are no-ops for
groups of size one, so single-process code paths need no special casing.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import state


def _size(group) -> int:
    if group is None or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def _rank(group) -> int:
    return dist.get_rank(group) if (group is not None and dist.is_initialized()) else 0


def _tp(group):
    if group is not None:
        return group
    return state.get_tensor_model_parallel_group() if state.model_parallel_is_initialized() else None


# ------------------------------------------------------------------ raw collectives
def all_reduce_(x: torch.Tensor, group) -> torch.Tensor:
    if _size(group) > 1:
        dist.all_reduce(x, group=group)
    return x


def split_last(x: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    return x.chunk(n, dim=-1)[_rank(group)].contiguous()


def split_first(x: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    if x.shape[0] % n:
        raise ValueError(f"first dim {x.shape[0]} not divisible by group size {n}")
    k = x.shape[0] // n
    return x[_rank(group) * k:(_rank(group) + 1) * k].contiguous()


def gather_first(x: torch.Tensor, group, output_split_sizes: Optional[List[int]] = None) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    x = x.contiguous()
    if output_split_sizes is None:
        out = torch.empty((x.shape[0] * n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out
    out = torch.empty((sum(output_split_sizes),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather(list(torch.split(out, output_split_sizes, dim=0)), x, group=group)
    return out


def reduce_scatter_first(x: torch.Tensor, group, input_split_sizes: Optional[List[int]] = None) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    x = x.contiguous()
    if input_split_sizes is None:
        if x.shape[0] % n:
            raise ValueError(f"first dim {x.shape[0]} not divisible by group size {n}")
        out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out
    parts = list(torch.split(x, input_split_sizes, dim=0))
    out = torch.empty_like(parts[_rank(group)])
    dist.reduce_scatter(out, parts, group=group)
    return out


def gather_last(x: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    x = x.contiguous()
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=-1).contiguous()


def reduce_scatter_last(x: torch.Tensor, group) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    parts = [p.contiguous() for p in x.chunk(n, dim=-1)]
    out = torch.empty_like(parts[0])
    dist.reduce_scatter(out, parts, group=group)
    return out


# ------------------------------------------------------------------ autograd pairs
class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce_(g.contiguous().clone() if _size(ctx.group) > 1 else g, ctx.group), None


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return all_reduce_(x.contiguous().clone() if _size(group) > 1 else x, group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _ScatterLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return split_last(x, group)

    @staticmethod
    def backward(ctx, g):
        return gather_last(g, ctx.group), None


class _GatherLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return gather_last(x, group)

    @staticmethod
    def backward(ctx, g):
        return split_last(g, ctx.group), None


class _ScatterFirst(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return split_first(x, group)

    @staticmethod
    def backward(ctx, g):
        return gather_first(g, ctx.group), None


class _GatherFirst(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, tp_grad_reduce, sizes):
        ctx.group, ctx.reduce, ctx.sizes = group, tp_grad_reduce, sizes
        return gather_first(x, group, sizes)

    @staticmethod
    def backward(ctx, g):
        # If the consumer computed in a tensor-parallel way the incoming gradients are partial
        # sums: reduce-scatter.  Otherwise every rank holds the same gradient: just split.
        if ctx.reduce:
            return reduce_scatter_first(g, ctx.group, ctx.sizes), None, None, None
        if ctx.sizes is not None:
            return torch.split(g, ctx.sizes, dim=0)[_rank(ctx.group)].contiguous(), None, None, None
        return split_first(g, ctx.group), None, None, None


class _ReduceScatterFirst(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, sizes):
        ctx.group, ctx.sizes = group, sizes
        return reduce_scatter_first(x, group, sizes)

    @staticmethod
    def backward(ctx, g):
        return gather_first(g, ctx.group, ctx.sizes), None, None


class _GatherLastRS(torch.autograd.Function):
    """all-gather(last) whose backward is reduce-scatter(last)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return gather_last(x, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_last(g, ctx.group), None


class _ReduceScatterLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_last(x, group)

    @staticmethod
    def backward(ctx, g):
        return gather_last(g, ctx.group), None


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, output_split_sizes, input_split_sizes):
        ctx.group, ctx.o, ctx.i = group, output_split_sizes, input_split_sizes
        n = _size(group)
        if n == 1:
            return x
        x = x.contiguous()
        if output_split_sizes is None:
            out = torch.empty_like(x)
        else:
            out = torch.empty((sum(output_split_sizes),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x, output_split_sizes=output_split_sizes, input_split_sizes=input_split_sizes,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return _AllToAll.apply(g, ctx.group, ctx.i, ctx.o), None, None, None


# ------------------------------------------------------------------ public wrappers
def copy_to_tensor_model_parallel_region(x, group=None): return _Copy.apply(x, _tp(group))
def reduce_from_tensor_model_parallel_region(x, group=None): return _Reduce.apply(x, _tp(group))
def scatter_to_tensor_model_parallel_region(x, group=None): return _ScatterLast.apply(x, _tp(group))
def gather_from_tensor_model_parallel_region(x, group=None): return _GatherLast.apply(x, _tp(group))
def scatter_to_sequence_parallel_region(x, group=None): return _ScatterFirst.apply(x, _tp(group))


def gather_from_sequence_parallel_region(x, tensor_parallel_output_grad: bool = True, group=None,
                                         output_split_sizes=None):
    return _GatherFirst.apply(x, _tp(group), tensor_parallel_output_grad, output_split_sizes)


def reduce_scatter_to_sequence_parallel_region(x, group=None, input_split_sizes=None):
    return _ReduceScatterFirst.apply(x, _tp(group), input_split_sizes)


def all_gather_last_dim_from_tensor_parallel_region(x, group=None): return _GatherLastRS.apply(x, _tp(group))
def reduce_scatter_last_dim_to_tensor_parallel_region(x, group=None): return _ReduceScatterLast.apply(x, _tp(group))


def all_to_all(group, x, output_split_sizes=None, input_split_sizes=None):
    return _AllToAll.apply(x, group, output_split_sizes, input_split_sizes)


def all_to_all_sp2hp(x, group=None):
    """[s/tp, h] -> [s, h/tp]: trade sequence sharding for hidden sharding
    (reference: mappings.py:541)."""
    group = _tp(group)
    n = _size(group)
    if n == 1:
        return x
    x2 = x.reshape(-1, x.shape[-1])
    send = torch.cat([c.contiguous() for c in x2.chunk(n, dim=1)], dim=0)
    return all_to_all(group, send)


def all_to_all_hp2sp(x, group=None):
    """[s, h/tp] -> [s/tp, h] (reference: mappings.py:570)."""
    group = _tp(group)
    n = _size(group)
    if n == 1:
        return x
    x2 = x.reshape(-1, x.shape[-1])
    recv = all_to_all(group, x2)
    return torch.cat(recv.chunk(n, dim=0), dim=1).contiguous()
