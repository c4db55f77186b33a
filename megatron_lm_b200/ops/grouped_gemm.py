"""Ragged grouped linear for MoE experts: rows of ``x`` are sorted by expert and expert ``e``
owns ``tokens_per_expert[e]`` consecutive rows (reference call site:
megatron/core/transformer/moe/experts.py:271-284, ``gg.ops.gmm``).

Each expert's product runs on the tcgen05 GEMM over a row slice - forward ``x_e W_e^T``,
data gradient ``dy_e W_e`` and weight gradient ``dy_e^T x_e`` accumulated in fp32 into the
expert's slice of ``weight.main_grad`` - so no operand is copied or transposed.  The split
sizes are read on the host once per call (the dispatcher already needs them for the
all-to-all split sizes).
"""
from __future__ import annotations

from typing import List, Sequence, Union

import torch

from .gemm import gemm
from .grad import deliver, has_main_grad, notify_ready


def _splits(tokens_per_expert) -> List[int]:
    if torch.is_tensor(tokens_per_expert):
        return [int(v) for v in tokens_per_expert.tolist()]
    return [int(v) for v in tokens_per_expert]


class _GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, splits):
        E, out_f, in_f = weight.shape
        y = torch.empty(x.shape[0], out_f, dtype=x.dtype, device=x.device)
        o = 0
        for e, n in enumerate(splits):
            if n:
                gemm(x[o:o + n], weight[e], out=y[o:o + n])
            o += n
        ctx.save_for_backward(x, weight)
        ctx.splits = splits
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        splits = ctx.splits
        dy = dy.contiguous()
        dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
        direct = has_main_grad(weight) and weight.main_grad.dtype == torch.float32
        gw = weight.main_grad.view(weight.shape) if direct else torch.zeros(weight.shape, dtype=torch.float32,
                                                                             device=weight.device)
        o = 0
        for e, n in enumerate(splits):
            if n:
                if dx is not None:
                    gemm(dy[o:o + n], weight[e], b_mn=True, out=dx[o:o + n])
                if weight.requires_grad:
                    gemm(dy[o:o + n], x[o:o + n], a_mn=True, b_mn=True, out=gw[e], accumulate=True)
            o += n
        if direct:
            notify_ready(weight)
            return dx, None, None
        return dx, (deliver(weight, gw) if weight.requires_grad else None), None


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, tokens_per_expert) -> torch.Tensor:
    """x [N, in] (expert-sorted), weight [E, out, in] -> [N, out]."""
    splits = _splits(tokens_per_expert)
    if not x.is_cuda:
        outs, o = [], 0
        for e, n in enumerate(splits):
            outs.append(x[o:o + n] @ weight[e].t())
            o += n
        return torch.cat(outs, dim=0) if outs else x.new_zeros(0, weight.shape[1])
    return _GroupedLinearFn.apply(x.contiguous(), weight, splits)
