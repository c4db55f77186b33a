"""Sequence-parallel collectives fused into the tensor-parallel GEMMs over NVLink peer memory.

``FusedTP`` owns, per tensor-parallel group, a set of symmetric-memory buffers (mapped into every
rank of the group) and drives the two fused kernels of ``csrc/tp_fused.cu``:

* ``ag_gemm(x, w)``  : y = allgather_seq(x) @ op(w).  Also returns the gathered activation, which
  the caller keeps for the weight-gradient product - nothing is re-gathered in backward (the
  reference re-gathers: megatron/core/tensor_parallel/layers.py:507-520).
* ``gemm_rs(a, w)``  : reduce_scatter_seq(a @ op(w)) (+ residual), the partial sums travelling as
  peer stores from the GEMM epilogue.

Buffers: one activation staging shard (the kernel's peers read it), signal words (ready/done per
peer), two receive areas for the reduce-scatter (alternating, so a fast rank may already deliver
call n+1 while a slow one still sums call n) and their arrival counters.  All flags are monotonic
sequence numbers; nothing is reset between calls.

Peer mappings come from ``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged over
the group's store); only plain peer pointers are used - no NVLink-switch reduction objects.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib

# Only plain peer pointers are used; keep the allocator from also binding the buffers to an
# NVLink-switch multicast object (a rank that exits while bound can disturb the other ranks).
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

_lib.register_signatures({
    "mlb_ag_gemm": "ipppppiiiiiipliplipiippp",
    "mlb_gemm_rs": "iplplippiiiiplpliippp",
    "mlb_gemm_rs_arrivals": "iii",
    "mlb_tp_fused_uses_pair": "iii",
    "mlb_occupy_sms": "iiip",
})


def _ptr_array(ptrs: List[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


class FusedTP:
    def __init__(self, group, rows_per_rank: int, max_k: int, max_n: int, dtype=torch.bfloat16,
                 n_comm: Optional[int] = None, dynamic_schedule: bool = True):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows = rows_per_rank
        if rows_per_rank % 128:
            raise ValueError("fused TP kernels need (seq * micro_batch / tp) to be a multiple of 128")
        self.dtype = dtype
        # copy-worker CTAs of the all-gather mode (each keeps 160 KB of peer reads in flight).  Sixteen instead of
        # eight at tensor-parallel 4 measured the same step (64,913 against 64,064 tokens/s) and the same kernel times.
        self.n_comm = n_comm if n_comm is not None else 8
        dev = torch.device("cuda", torch.cuda.current_device())
        self.max_k, self.max_n = max_k, max_n
        bpr = rows_per_rank // 128
        # one symmetric allocation, carved up: [x shard | recv 0 | recv 1 | words]
        x_bytes = rows_per_rank * max_k * 2
        recv_bytes = self.tp * rows_per_rank * max_n * 2
        words = 2 * self.tp + 2 * bpr + 64
        self._offs = (0, x_bytes, x_bytes + recv_bytes, x_bytes + 2 * recv_bytes)
        total = x_bytes + 2 * recv_bytes + words * 4
        total = (total + 1023) // 1024 * 1024
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize()
        self.hdl = symm_mem.rendezvous(self.buf, group)
        base = [int(p) for p in self.hdl.buffer_ptrs]
        self.x_ptrs = [b + self._offs[0] for b in base]
        self.recv_ptrs = [[b + self._offs[1] for b in base], [b + self._offs[2] for b in base]]
        w0 = self._offs[3]
        self.sig_ptrs = [b + w0 for b in base]                               # ready[tp], done[tp]
        self.cnt_ptrs = [[b + w0 + 4 * (2 * self.tp) for b in base],         # counters of recv 0
                         [b + w0 + 4 * (2 * self.tp + bpr) for b in base]]   # counters of recv 1
        self.x_local = self.buf[self._offs[0]:self._offs[0] + x_bytes].view(dtype)
        self.chunk_flags = torch.zeros(self.tp * bpr, dtype=torch.int32, device=dev)
        self.comm_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        # {next tile, pairs that have left} of the dynamic tile schedule; the kernel leaves both at zero
        self.sched = torch.zeros(2, dtype=torch.int32, device=dev) if dynamic_schedule else None
        self.ag_seq = 0
        self.comm_total = 0
        self.rs_calls = 0
        self.cnt_expected = [0, 0]
        self.hdl.barrier()

    # ------------------------------------------------------------------ all-gather -> GEMM
    def ag_gemm(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                b_mn: bool = False, out_dtype=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """x: this rank's [rows_per_rank, K] shard.  weight: [N, K] (``b_mn=False``) or stored [K, N].
        Returns (y [tp*rows, N], gathered [tp*rows, K])."""
        x2 = x.reshape(-1, x.shape[-1])
        rows, K = x2.shape
        assert rows == self.rows and K <= self.max_k and x2.dtype == self.dtype
        N = weight.shape[1] if b_mn else weight.shape[0]
        xs = self.x_local[:rows * K].view(rows, K)
        xs.copy_(x2)
        gathered = torch.empty(self.tp * rows, K, dtype=self.dtype, device=x.device)
        y = torch.empty(self.tp * rows, N, dtype=out_dtype or self.dtype, device=x.device)
        self.ag_seq += 1
        self.comm_total += self.n_comm
        st = _lib.status_word()
        mode = 0 if y.dtype != torch.float32 else 1
        bias_c = None if bias is None else bias.to(self.dtype).contiguous()
        _lib.check(_lib.lib().mlb_ag_gemm(
            1 if self.dtype == torch.bfloat16 else 0, _ptr_array(self.x_ptrs), _ptr_array(self.sig_ptrs),
            gathered.data_ptr(), self.chunk_flags.data_ptr(), self.comm_counter.data_ptr(), self.rank, self.tp,
            rows, self.ag_seq, self.comm_total, self.n_comm, weight.data_ptr(), weight.stride(0), int(b_mn), y.data_ptr(),
            y.stride(0), mode, _lib.ptr(bias_c), N, K, st.data_ptr(), _lib.stream(), _lib.ptr(self.sched)), "ag_gemm")
        return y, gathered

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_rs(self, a: torch.Tensor, weight: torch.Tensor, b_mn: bool = False,
                residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """a: [tp*rows_per_rank, K_local].  Returns this rank's [rows_per_rank, N] slice of the summed product."""
        a2 = a.reshape(-1, a.shape[-1])
        if a2.stride(1) != 1:
            a2 = a2.contiguous()
        M, K = a2.shape
        assert M == self.tp * self.rows
        N = weight.shape[1] if b_mn else weight.shape[0]
        assert N <= self.max_n
        which = self.rs_calls & 1
        self.rs_calls += 1
        L = _lib.lib()
        self.cnt_expected[which] += L.mlb_gemm_rs_arrivals(self.tp, N, self.rows)
        out = torch.empty(self.rows, N, dtype=self.dtype, device=a.device)
        res2 = None if residual is None else residual.reshape(self.rows, N)
        st = _lib.status_word()
        _lib.check(L.mlb_gemm_rs(
            1 if self.dtype == torch.bfloat16 else 0, a2.data_ptr(), a2.stride(0), weight.data_ptr(), weight.stride(0),
            int(b_mn), _ptr_array(self.recv_ptrs[which]), _ptr_array(self.cnt_ptrs[which]), self.cnt_expected[which],
            self.rank, self.tp, self.rows, _lib.ptr(res2), 0 if res2 is None else res2.stride(0), out.data_ptr(),
            out.stride(0), N, K, st.data_ptr(), _lib.stream(), _lib.ptr(self.sched)), "gemm_rs")
        return out


def occupy_sms(n_ctas: int, smem_bytes: int, usec: int, stream=None) -> None:
    """Test aid: hold ``n_ctas`` SMs' worth of shared memory on ``stream`` for ``usec`` microseconds (capped at
    0.5 s) - a stand-in for long-running kernels of other streams that keep SMs away from a fused kernel."""
    st = (stream or torch.cuda.current_stream()).cuda_stream
    _lib.stream()
    _lib.check(_lib.lib().mlb_occupy_sms(n_ctas, smem_bytes, usec, st), "occupy_sms")


def attach_fused_tp(model_chunks, config, seq_length: int, micro_batch_size: int) -> Optional[FusedTP]:
    """Create one FusedTP for the tensor-parallel group and hand it to every TP linear of the model."""
    from ..parallel import state
    from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
    tp = state.get_tensor_model_parallel_world_size()
    if tp == 1 or not config.sequence_parallel:
        return None
    rows = seq_length * micro_batch_size // config.context_parallel_size // tp
    if rows % 128:
        return None
    # Other kernels may hold SMs for a long time while these run (NCCL send / receive kernels of a pipeline stage,
    # gradient reductions of a data-parallel group), so part of a fused kernel's grid can be waiting for an SM.
    # The CTA-pair kernel hands tiles to running blocks only (dynamic schedule) and tolerates that; the single-CTA
    # kernel assigns tiles to block numbers up front and is used only when nothing else competes for SMs.
    shared_sms = state.get_pipeline_model_parallel_world_size() > 1 or state.get_data_parallel_world_size() > 1
    if shared_sms and not _lib.lib().mlb_tp_fused_uses_pair(rows, 256, 8):
        return None
    max_k = max_n = 0
    lins = []
    for chunk in model_chunks:
        for m in chunk.modules():
            if isinstance(m, ColumnParallelLinear) and m.sequence_parallel and m.weight is not None:
                # forward AG over K = input_size; backward RS delivers N = input_size
                max_k = max(max_k, m.input_size)
                max_n = max(max_n, m.input_size)
                lins.append(m)
            elif isinstance(m, RowParallelLinear) and m.sequence_parallel:
                # forward RS delivers N = output_size; backward AG over K = output_size
                max_n = max(max_n, m.output_size)
                max_k = max(max_k, m.output_size)
                lins.append(m)
    if not lins:
        return None
    fused = FusedTP(state.get_tensor_model_parallel_group(), rows, max_k, max_n, config.params_dtype)
    for m in lins:
        m.fused = fused
    return fused


def detach_fused_tp(model_chunks) -> None:
    """Take the fused communicator off every layer again: they go back to NCCL collectives around plain GEMMs."""
    for chunk in model_chunks:
        for m in chunk.modules():
            if getattr(m, "fused", None) is not None:
                m.fused = None
