"""Ragged grouped linear for MoE experts: rows of ``x`` are sorted by expert and expert ``e``
owns ``tokens_per_expert[e]`` consecutive rows (reference call site:
megatron/core/transformer/moe/experts.py:271-284, ``gg.ops.gmm``).

Forward ``x_e W_e^T`` and data gradient ``dy_e W_e`` of all experts run as ONE launch of the tcgen05
GEMM in its grouped mode: a device table of row tiles (begin, end, expert), at most 128 rows each and
never spanning two experts, replaces the regular tile grid; B is the stacked expert weights addressed
with the expert's row offset.  The weight gradient ``dy_e^T x_e`` reduces over an expert's rows, so it
runs per expert (the reduction range must end exactly at the expert boundary), accumulating in fp32
into the expert's slice of ``weight.main_grad``.  No operand is copied or transposed.  The split sizes
are read on the host once per call (the dispatcher already needs them for the all-to-all splits).
"""
from __future__ import annotations

from typing import List, Sequence, Union

import torch

from . import _lib
from .gemm import gemm
from .grad import deliver, has_main_grad, notify_ready

_lib.register_signatures({"mlb_gemm_grouped": "iplplipl" "piiiii" "pp"})


def build_tile_table(splits: Sequence[int], device) -> torch.Tensor:
    """int32 [n_tiles, 4] records (row_begin, row_end, expert, 0)."""
    recs, o = [], 0
    for e, n in enumerate(splits):
        for r in range(o, o + n, 128):
            recs.append((r, min(r + 128, o + n), e, 0))
        o += n
    return torch.tensor(recs, dtype=torch.int32).reshape(-1, 4).to(device, non_blocking=True)


def grouped_gemm(a: torch.Tensor, weight: torch.Tensor, tiles: torch.Tensor, b_mn: bool) -> torch.Tensor:
    """a [T, K] rows sorted by expert; weight [E, out, in].  ``b_mn=False``: a @ W_e^T -> [T, out];
    ``b_mn=True``: a @ W_e -> [T, in]."""
    E, out_f, in_f = weight.shape
    T = a.shape[0]
    N, K = (in_f, out_f) if b_mn else (out_f, in_f)
    y = torch.empty(T, N, dtype=a.dtype, device=a.device)
    if tiles.shape[0] == 0:
        return y
    st = _lib.status_word()
    _lib.check(_lib.lib().mlb_gemm_grouped(1 if a.dtype == torch.bfloat16 else 0, a.data_ptr(), a.stride(0),
                                           weight.data_ptr(), weight.stride(1), int(b_mn), y.data_ptr(), y.stride(0),
                                           tiles.data_ptr(), tiles.shape[0], E, T, N, K, st.data_ptr(), _lib.stream()),
               "gemm_grouped")
    return y


def _splits(tokens_per_expert) -> List[int]:
    if torch.is_tensor(tokens_per_expert):
        return [int(v) for v in tokens_per_expert.tolist()]
    return [int(v) for v in tokens_per_expert]


class _GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, splits):
        E, out_f, in_f = weight.shape
        tiles = build_tile_table(splits, x.device)
        w = weight if weight.is_contiguous() else weight.contiguous()
        y = grouped_gemm(x, w, tiles, False)
        ctx.save_for_backward(x, weight, tiles)
        ctx.splits = splits
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, tiles = ctx.saved_tensors
        splits = ctx.splits
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            if weight.shape[1] % 64 == 0:
                dx = grouped_gemm(dy, weight if weight.is_contiguous() else weight.contiguous(), tiles, True)
            else:
                dx = torch.empty_like(x)
        loop_dx = dx is not None and weight.shape[1] % 64 != 0
        direct = has_main_grad(weight) and weight.main_grad.dtype == torch.float32
        gw = weight.main_grad.view(weight.shape) if direct else torch.zeros(weight.shape, dtype=torch.float32,
                                                                             device=weight.device)
        o = 0
        for e, n in enumerate(splits):
            if n:
                if loop_dx:
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
