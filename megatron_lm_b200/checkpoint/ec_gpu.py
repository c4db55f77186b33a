"""Erasure-coded in-memory checkpoint on GPUs: parity computed as a reduction over peer memory.

Every rank of the group keeps, in one symmetric-memory allocation that all ranks of the node can address,
(1) a device snapshot of its state bytes and (2) the parity chunks it owns.  Encoding is ONE kernel launch
per rank (``csrc/ec.cu`` batched form): for every stripe whose first parity slot this rank owns it pulls the
k member chunks from the peers' snapshots over NVLink, multiplies by the generator rows in GF(2^8), keeps
parity 0 and stores the other parities straight into their owners' memory - each data byte crosses NVLink
once.  A second tier copies snapshot and parity to pinned host memory on a side stream
(``cudaMemcpyAsync``), so a GPU whose memory is gone can be rebuilt from the survivors' GPUs and, failing
that, from their hosts.  Decoding is the same kernel with rows of the inverted survivor matrix, launched by
the rank that lost data.

This is the GPU counterpart of ``ec_checkpoint.ECCheckpointManager`` (same stripe plan, same generator, same
decode algebra, byte-identical results); the reference only replicates
(megatron/training/checkpointing.py:520-544).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..ops import _lib
from . import gf256
from .ec_plan import StripePlan, plan_stripes

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

_lib.register_signatures({"mlb_ec_apply_batch": "pilip", "mlb_ec_job_bytes": "",
                          "mlb_ec_apply_batch_staged": "piliipp", "mlb_stream_copy": "pplip"})

_JOB = np.dtype([("src", "<u8", 16), ("dst", "<u8", 4), ("coef", "u1", (4, 16)), ("k", "<i4"), ("m", "<i4"),
                 ("pad", "<i4", 2)])


class GpuECCheckpoint:
    def __init__(self, group, state_bytes: int, k: Optional[int] = None, m: int = 2, chunk_bytes: int = 1 << 20,
                 host_tier: bool = True, encode_blocks: int = 0, staged: bool = True, host_copy: str = "kernel",
                 host_copy_blocks: int = 4):
        import torch.distributed._symmetric_memory as symm_mem
        assert _JOB.itemsize == _lib.lib().mlb_ec_job_bytes()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.m = m
        self.k = k if k is not None else self.world - m
        if self.k + self.m > self.world:
            raise ValueError("the GPU tier needs k + m <= group size")
        self.chunk = int(chunk_bytes)
        self.encode_blocks = encode_blocks
        self.staged = staged
        # "kernel": a few thread blocks store the snapshot and parity into pinned host memory; "dma": cudaMemcpyAsync
        # (the copy engine then also serves the training stream's device-to-host reads one after the other)
        self.host_copy = host_copy
        self.host_copy_blocks = host_copy_blocks
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        n = torch.tensor([(state_bytes + self.chunk - 1) // self.chunk], dtype=torch.int64, device=dev)
        dist.all_reduce(n, op=dist.ReduceOp.MAX, group=group)
        self.n_chunks = int(n.item())
        self.plan: StripePlan = plan_stripes(self.world, self.k, self.m, self.n_chunks)
        self.G = gf256.generator_matrix(self.k, self.m)
        # parity slots: (stripe, parity index) -> slot on its owner
        self.slot: Dict[Tuple[int, int], int] = {}
        counts = [0] * self.world
        for s in self.plan.stripes:
            for i, o in enumerate(s.parity_owners):
                self.slot[(s.index, i)] = counts[o]
                counts[o] += 1
        self.parity_off = self.n_chunks * self.chunk
        total = self.parity_off + max(counts) * self.chunk
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize()
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.base = [int(p) for p in self.hdl.buffer_ptrs]
        self.n_parity = counts[self.rank]
        self.state_bytes = state_bytes
        self.iteration: Optional[int] = None
        self.stream = torch.cuda.Stream()
        self.host = torch.empty(total, dtype=torch.uint8, pin_memory=True) if host_tier else None
        self.host_event = None
        self._encode_jobs = self._build_encode_jobs()
        self._decode_cache: Dict = {}
        self.stats: Dict[str, float] = {}
        self.hdl.barrier()

    # -- addresses ---------------------------------------------------------------------
    def _data_addr(self, rank: int, chunk: int) -> int:
        return self.base[rank] + chunk * self.chunk

    def _parity_addr(self, stripe: int, i: int) -> int:
        owner = self.plan.stripes[stripe].parity_owners[i]
        return self.base[owner] + self.parity_off + self.slot[(stripe, i)] * self.chunk

    def _to_device(self, jobs: np.ndarray) -> torch.Tensor:
        return torch.from_numpy(jobs.view(np.uint8).reshape(-1).copy()).to(self.dev)

    def _build_encode_jobs(self):
        mine = [s for s in self.plan.stripes if s.parity_owners[0] == self.rank]
        jobs = np.zeros(len(mine), dtype=_JOB)
        for n, s in enumerate(mine):
            for pos, (r, c) in enumerate(s.data):
                jobs[n]["src"][pos] = self._data_addr(r, c)
                for i in range(self.m):
                    jobs[n]["coef"][i][pos] = self.G[i, pos]
            for i in range(self.m):
                jobs[n]["dst"][i] = self._parity_addr(s.index, i)
            jobs[n]["k"], jobs[n]["m"] = len(s.data), self.m
        return (self._to_device(jobs), len(mine)) if len(mine) else (None, 0)

    def _launch(self, jobs):
        tbl, n = jobs
        if not n:
            return
        st = torch.cuda.current_stream().cuda_stream
        if self.staged and self.chunk % 4096 == 0:
            # sources staged through shared memory by bulk copies (large NVLink requests, several in flight per SM)
            _lib.check(_lib.lib().mlb_ec_apply_batch_staged(tbl.data_ptr(), n, self.chunk, max(self.k, 1), self.encode_blocks,
                                                            _lib.status_word().data_ptr(), st), "ec batch")
        else:
            _lib.check(_lib.lib().mlb_ec_apply_batch(tbl.data_ptr(), n, self.chunk, self.encode_blocks, st), "ec batch")

    # -- save ---------------------------------------------------------------------------
    def save(self, tensors: Sequence[torch.Tensor], iteration: int, overlap: bool = False) -> Dict[str, float]:
        """Snapshot + encode (+ host tier).  With ``overlap`` the encode and the host copies run on the manager's
        side stream and this call returns after the snapshot; ``wait()`` joins them."""
        cur = torch.cuda.current_stream()
        cur.wait_stream(self.stream)                    # a previous overlapped encode / host copy still reads the snapshot
        if getattr(self, "_events", None) is not None and overlap:
            # device times of the previous (overlapped) save, complete by now
            pe = self._events
            if pe[3].query():
                self.stats = {"snapshot_ms": pe[0].elapsed_time(pe[1]), "encode_ms": pe[2].elapsed_time(pe[3]),
                              "bytes": self.stats.get("bytes", 0.0), "of_iteration": float(self.iteration or 0)}
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        e[0].record(cur)
        o = 0
        for t in tensors:
            b = t.detach().contiguous().view(-1).view(torch.uint8)
            self.buf[o:o + b.numel()].copy_(b, non_blocking=True)
            o += b.numel()
        if o > self.n_chunks * self.chunk:
            raise ValueError("state is larger than the size this manager was created for")
        e[1].record(cur)
        self.hdl.barrier()                              # every rank's snapshot is in place
        st = self.stream if overlap else cur
        st.wait_stream(cur)
        with torch.cuda.stream(st):
            e[2].record(st)
            self._launch(self._encode_jobs)
            e[3].record(st)
            self.hdl.barrier()                          # parities (also those stored by peers) are complete
        if self.host is not None:
            self.stream.wait_stream(st)
            with torch.cuda.stream(self.stream):
                total = self.buf.numel()
                if self.host_copy == "kernel" and total % 16 == 0:
                    _lib.check(_lib.lib().mlb_stream_copy(self.host.data_ptr(), self.buf.data_ptr(), total,
                                                          self.host_copy_blocks, self.stream.cuda_stream), "stream_copy")
                else:
                    self.host.copy_(self.buf, non_blocking=True)
                self.host_event = torch.cuda.Event()
                self.host_event.record(self.stream)
        self.iteration = iteration
        self._events = e
        if not overlap:
            torch.cuda.synchronize()
            self.stats = {"snapshot_ms": e[0].elapsed_time(e[1]), "encode_ms": e[2].elapsed_time(e[3]),
                          "bytes": float(o)}
        else:
            self.stats = dict(self.stats, bytes=float(o))
        return self.stats

    def wait(self):
        torch.cuda.current_stream().wait_stream(self.stream)
        if self.host_event is not None:
            self.host_event.synchronize()

    # -- failure simulation / recovery -----------------------------------------------------
    def drop_device_state(self):
        """What a replacement GPU starts with: nothing in device memory."""
        self.wait()                  # the last save's parity kernels (this rank's and the peers', behind its barrier)
        self.buf.zero_()
        torch.cuda.synchronize()

    def restore_from_host(self):
        """Second tier: refill this rank's device snapshot and parity from its pinned host copy."""
        if self.host is None:
            raise RuntimeError("no host tier")
        self.wait()
        self.buf.copy_(self.host, non_blocking=True)

    def recover(self, lost_ranks: Sequence[int], tensors_out: Optional[Sequence[torch.Tensor]] = None) -> int:
        """All ranks call.  Ranks in ``lost_ranks`` rebuild their data and parity chunks from k surviving members
        of each stripe; then every rank copies its snapshot back into ``tensors_out`` (roll-back)."""
        lost = sorted(set(int(r) for r in lost_ranks))
        if len(lost) > self.m:
            raise RuntimeError(f"{len(lost)} ranks lost but the code tolerates {self.m}")
        self.wait()                                     # an overlapped encode / host copy of the last save
        self.hdl.barrier()
        if self.rank in lost:
            jobs = []
            k, m = self.k, self.m
            for s in self.plan.stripes:
                kk = len(s.data)
                lost_data = [pos for pos, (r, _) in enumerate(s.data) if r in lost]
                lost_par = [i for i, o in enumerate(s.parity_owners) if o in lost]
                my_data = [pos for pos in lost_data if s.data[pos][0] == self.rank]
                my_par = [i for i in lost_par if s.parity_owners[i] == self.rank]
                if not my_data and not my_par:
                    continue
                present = [pos for pos in range(kk) if pos not in lost_data] + list(range(kk, k)) + \
                    [k + i for i in range(m) if i not in lost_par]
                wanted = my_data + [k + i for i in my_par]
                key = (kk, tuple(present), tuple(wanted))
                if key not in self._decode_cache:
                    self._decode_cache[key] = gf256.decode_matrix(k, m, present, wanted)
                M, use = self._decode_cache[key]
                for w_i, w in enumerate(wanted):
                    job = np.zeros((), dtype=_JOB)
                    n_src = 0
                    for u_i, u in enumerate(use):
                        coef = int(M[w_i, u_i])
                        if coef == 0 or kk <= u < k:                    # absent members of a short stripe are zeros
                            continue
                        if u < kk:
                            r, c = s.data[u]
                            job["src"][n_src] = self._data_addr(r, c)
                        else:
                            job["src"][n_src] = self._parity_addr(s.index, u - k)
                        job["coef"][0][n_src] = coef
                        n_src += 1
                    job["dst"][0] = self._data_addr(self.rank, s.data[w][1]) if w < k else self._parity_addr(s.index, w - k)
                    job["k"], job["m"] = n_src, 1
                    jobs.append(job)
            if jobs:
                arr = np.array(jobs, dtype=_JOB)
                self._launch((self._to_device(arr), len(jobs)))
        torch.cuda.synchronize()
        self.hdl.barrier()
        if tensors_out is not None:
            o = 0
            for t in tensors_out:
                n = t.numel() * t.element_size()
                t.detach().view(-1).view(torch.uint8).copy_(self.buf[o:o + n])
                o += n
        return self.iteration if self.iteration is not None else -1
