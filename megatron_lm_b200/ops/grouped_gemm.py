"""Ragged grouped linear for MoE experts: rows of ``x`` are sorted by expert and expert ``e``
owns ``tokens_per_expert[e]`` consecutive rows (reference call site:
megatron/core/transformer/moe/experts.py:271-284, ``gg.ops.gmm``).

Forward ``x_e W_e^T`` and data gradient ``dy_e W_e`` of all experts run as ONE launch of the tcgen05
GEMM in its grouped mode: a device table of row tiles (begin, end, expert), at most 128 rows each and
never spanning two experts, replaces the regular tile grid; B is the stacked expert weights addressed
with the expert's row offset.  The weight gradient ``dy_e^T x_e`` of all experts is ONE launch too: output
tiles are numbered per expert, each reduces over its expert's rows, and the rows of the last reduction
step that belong to the next expert are cleared in shared memory before the MMA (both operands are read
MN-major where they are; fp32 accumulation straight into ``weight.main_grad``).  No operand is copied or
transposed.  When the per-expert token counts arrive as a device tensor, the tile table and the expert
offsets are built by a small kernel and the GEMMs read the tile count from device memory: the host never
waits for the routing result (the reference synchronises here:
megatron/core/transformer/moe/token_dispatcher.py:406-420).
"""
from __future__ import annotations

from typing import List, Sequence, Union

import torch

from . import _lib
from .gemm import gemm
from .grad import deliver, has_main_grad, notify_ready

_lib.register_signatures({"mlb_gemm_grouped": "iplplipl" "piiiii" "ppp",
                          "mlb_moe_tile_table": "pipippp",
                          "mlb_gemm_grouped_wgrad": "iplplppiiiiipp"})


class TileTable:
    """Row tiles of a grouped GEMM.  ``tiles`` int32 [cap, 4]; ``count`` None (all records valid) or a device
    int32 [1]; ``offsets`` device int32 [E + 1] (expert row boundaries) or None; ``splits`` host list or None."""

    def __init__(self, tiles, count=None, offsets=None, splits=None):
        self.tiles, self.count, self.offsets, self.splits = tiles, count, offsets, splits


def build_tile_table_device(tokens_per_expert: torch.Tensor, total_rows: int) -> TileTable:
    """Tile table from device-resident counts, without a host read: capacity ceil(T / 128) + E records."""
    E = tokens_per_expert.numel()
    cap = (total_rows + 127) // 128 + E
    dev = tokens_per_expert.device
    tiles = torch.empty(cap, 4, dtype=torch.int32, device=dev)
    count = torch.empty(1, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    c64 = tokens_per_expert.to(torch.int64).contiguous()
    _lib.check(_lib.lib().mlb_moe_tile_table(c64.data_ptr(), E, tiles.data_ptr(), cap, count.data_ptr(),
                                             offsets.data_ptr(), _lib.stream()), "moe_tile_table")
    return TileTable(tiles, count, offsets, None)


def build_tile_table(splits: Sequence[int], device) -> torch.Tensor:
    """int32 [n_tiles, 4] records (row_begin, row_end, expert, 0)."""
    recs, o = [], 0
    for e, n in enumerate(splits):
        for r in range(o, o + n, 128):
            recs.append((r, min(r + 128, o + n), e, 0))
        o += n
    return torch.tensor(recs, dtype=torch.int32).reshape(-1, 4).to(device, non_blocking=True)


def grouped_gemm(a: torch.Tensor, weight: torch.Tensor, tiles, b_mn: bool) -> torch.Tensor:
    """a [T, K] rows sorted by expert; weight [E, out, in].  ``b_mn=False``: a @ W_e^T -> [T, out];
    ``b_mn=True``: a @ W_e -> [T, in].  ``tiles``: a :class:`TileTable` or a plain int32 [n, 4] tensor."""
    tt = tiles if isinstance(tiles, TileTable) else TileTable(tiles)
    E, out_f, in_f = weight.shape
    T = a.shape[0]
    N, K = (in_f, out_f) if b_mn else (out_f, in_f)
    y = torch.empty(T, N, dtype=a.dtype, device=a.device)
    if tt.tiles.shape[0] == 0:
        return y
    st = _lib.status_word()
    _lib.check(_lib.lib().mlb_gemm_grouped(1 if a.dtype == torch.bfloat16 else 0, a.data_ptr(), a.stride(0),
                                           weight.data_ptr(), weight.stride(1), int(b_mn), y.data_ptr(), y.stride(0),
                                           tt.tiles.data_ptr(), tt.tiles.shape[0], E, T, N, K, st.data_ptr(),
                                           _lib.stream(), _lib.ptr(tt.count)), "gemm_grouped")
    return y


def grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor,
                  accumulate: bool) -> None:
    """out [E, N_out, K_in] fp32 (=|+=) dy_e^T x_e for every expert in one launch; ``offsets`` int32 [E + 1]."""
    E, n_out, k_in = out.shape
    st = _lib.status_word()
    _lib.check(_lib.lib().mlb_gemm_grouped_wgrad(1 if dy.dtype == torch.bfloat16 else 0, dy.data_ptr(), dy.stride(0),
                                                 x.data_ptr(), x.stride(0), out.data_ptr(), offsets.data_ptr(), E,
                                                 dy.shape[0], n_out, k_in, int(accumulate), st.data_ptr(),
                                                 _lib.stream()), "gemm_grouped_wgrad")


def _splits(tokens_per_expert) -> List[int]:
    if torch.is_tensor(tokens_per_expert):
        return [int(v) for v in tokens_per_expert.tolist()]
    return [int(v) for v in tokens_per_expert]


class _GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, tokens_per_expert):
        E, out_f, in_f = weight.shape
        if torch.is_tensor(tokens_per_expert) and tokens_per_expert.is_cuda:
            table = build_tile_table_device(tokens_per_expert, x.shape[0])       # no host read of the counts
        else:
            splits = _splits(tokens_per_expert)
            off = torch.tensor([0] + list(torch.tensor(splits).cumsum(0).tolist()), dtype=torch.int32)
            table = TileTable(build_tile_table(splits, x.device), None, off.to(x.device, non_blocking=True), splits)
        w = weight if weight.is_contiguous() else weight.contiguous()
        y = grouped_gemm(x, w, table, False)
        ctx.save_for_backward(x, weight)
        ctx.table = table
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        table = ctx.table
        dy = dy.contiguous()
        E, out_f, in_f = weight.shape
        one_launch_dx = out_f % 64 == 0
        one_launch_dw = out_f % 128 == 0 and in_f % 4 == 0 and table.offsets is not None
        splits = None
        if not (one_launch_dx and one_launch_dw):
            # shapes outside the one-launch kernels: per-expert products need the split sizes on the host
            splits = table.splits if table.splits is not None else \
                [int(v) for v in (table.offsets[1:] - table.offsets[:-1]).tolist()]
        dx = None
        if ctx.needs_input_grad[0]:
            if one_launch_dx:
                dx = grouped_gemm(dy, weight if weight.is_contiguous() else weight.contiguous(), table, True)
            else:
                dx = torch.empty_like(x)
                o = 0
                for e, n in enumerate(splits):
                    if n:
                        gemm(dy[o:o + n], weight[e], b_mn=True, out=dx[o:o + n])
                    o += n
        if not weight.requires_grad:
            return dx, None, None
        direct = has_main_grad(weight) and weight.main_grad.dtype == torch.float32
        gw = weight.main_grad.view(weight.shape) if direct else torch.empty(weight.shape, dtype=torch.float32,
                                                                             device=weight.device)
        if one_launch_dw:
            grouped_wgrad(dy, x, gw, table.offsets, accumulate=direct)
        else:
            if not direct:
                gw.zero_()
            o = 0
            for e, n in enumerate(splits):
                if n:
                    gemm(dy[o:o + n], x[o:o + n], a_mn=True, b_mn=True, out=gw[e], accumulate=True)
                o += n
        if direct:
            notify_ready(weight)
            return dx, None, None
        return dx, deliver(weight, gw), None


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, tokens_per_expert) -> torch.Tensor:
    """x [N, in] (expert-sorted), weight [E, out, in] -> [N, out].  ``tokens_per_expert``: host list, or a
    tensor; a CUDA tensor is consumed on the device (no synchronisation)."""
    if not x.is_cuda:
        splits = _splits(tokens_per_expert)
        outs, o = [], 0
        for e, n in enumerate(splits):
            outs.append(x[o:o + n] @ weight[e].t())
            o += n
        return torch.cat(outs, dim=0) if outs else x.new_zeros(0, weight.shape[1])
    return _GroupedLinearFn.apply(x.contiguous(), weight, tokens_per_expert)
