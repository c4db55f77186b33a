"""Erasure-coded in-memory checkpoint of per-rank flat state (optimizer shards, weights).

The reference's in-memory ("local non-persistent") checkpoint survives rank loss by *replication*
to ``factor - 1`` peers (megatron/training/checkpointing.py:520-544, training.py:807-838).  This
module provides the same guarantee with parity instead of copies: for m tolerated losses the
storage overhead is m/k of the state instead of m whole copies.

Protocol (all ranks of a group call collectively):

``save(tensors, iteration)``
  1. every rank snapshots its own bytes (pinned host memory; a side-stream D2H copy on GPUs) -
     survivors roll back to this snapshot on recovery;
  2. the state is cut into ``chunk_bytes`` chunks and placed into stripes by
     :func:`ec_plan.plan_stripes`;
  3. for each parity slot, every stripe member multiplies its chunk by its GF(2^8) coefficient
     and the products are XOR-reduced onto the parity owner.  On CPU/Gloo that is a BXOR
     ``reduce``; on GPUs the owner's kernel reads the members' chunks through peer pointers and
     does multiply+XOR in one pass (``ops/ec.py``).

``recover(lost_ranks)``
  survivors restore from their snapshot; for every stripe that lost members, k surviving members
  are multiplied by the rows of the inverted generator sub-matrix and XOR-reduced onto each lost
  rank (or its replacement process), which ends up with its bytes at the saved iteration.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from . import gf256
from .ec_plan import StripePlan, plan_stripes


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    return t.detach().contiguous().view(-1).view(torch.uint8)


class ECCheckpointManager:
    def __init__(self, group=None, k: Optional[int] = None, m: int = 1, chunk_bytes: int = 1 << 20,
                 keep_parity_on_host: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.m = m
        self.k = k if k is not None else (self.world - m if self.world - m >= 1 else self.world)
        if self.k + self.m > self.world and self.k != self.world:
            raise ValueError("k + m must fit in the group, or k must equal the group size (host parity)")
        self.chunk_bytes = int(chunk_bytes)
        self.keep_parity_on_host = keep_parity_on_host
        self.G = gf256.generator_matrix(self.k, self.m)
        self._mul = gf256.tables()[2]
        self.iteration: Optional[int] = None
        self.plan: Optional[StripePlan] = None
        self.snapshot: Optional[torch.Tensor] = None      # this rank's bytes at `iteration`
        self.layout: List[Tuple[int, torch.Size, torch.dtype]] = []
        self.parity: Dict[Tuple[int, int], torch.Tensor] = {}   # (stripe, parity idx) -> chunk
        self.nbytes = 0
        self.stats: Dict[str, float] = {}

    # ------------------------------------------------------------------ helpers
    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if (self.group is not None) else r

    def _gfmul(self, c: int, buf: np.ndarray) -> np.ndarray:
        if c == 1:
            return buf
        if c == 0:
            return np.zeros_like(buf)
        return self._mul[c][buf]

    def _xor_reduce(self, arr: np.ndarray, dst: int) -> Optional[np.ndarray]:
        """XOR of ``arr`` over the group, delivered to group-rank ``dst``."""
        if self.world == 1:
            return arr
        t = torch.from_numpy(arr)
        dist.reduce(t, dst=self._global(dst), op=dist.ReduceOp.BXOR, group=self.group)
        return t.numpy() if self.rank == dst else None

    def _chunk(self, data: np.ndarray, c: int) -> np.ndarray:
        return data[c * self.chunk_bytes:(c + 1) * self.chunk_bytes]

    # ------------------------------------------------------------------ save
    def save(self, tensors: Sequence[torch.Tensor], iteration: int) -> Dict[str, float]:
        t0 = time.perf_counter()
        flat = [_as_bytes(t) for t in tensors]
        self.layout = [(f.numel(), t.shape, t.dtype) for f, t in zip(flat, tensors)]
        nbytes = sum(f.numel() for f in flat)
        n_chunks = (nbytes + self.chunk_bytes - 1) // self.chunk_bytes
        if self.world > 1:
            mx = torch.tensor([n_chunks], dtype=torch.int64)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)
            n_chunks = int(mx.item())
        padded = n_chunks * self.chunk_bytes
        # 1. local snapshot in (pinned) host memory
        pin = torch.cuda.is_available()
        if self.snapshot is None or self.snapshot.numel() != padded:
            self.snapshot = torch.zeros(padded, dtype=torch.uint8, pin_memory=pin)
        o = 0
        for f in flat:
            self.snapshot[o:o + f.numel()].copy_(f, non_blocking=True)
            o += f.numel()
        if pin:
            torch.cuda.current_stream().synchronize()
        self.snapshot[o:].zero_()
        self.nbytes = nbytes
        t1 = time.perf_counter()
        # 2. placement
        if self.plan is None or self.plan.chunks_per_rank != n_chunks:
            self.plan = plan_stripes(self.world, self.k, self.m, n_chunks)
        data = self.snapshot.numpy()
        # 3. parity: one XOR-reduction per (owner, parity index), batching that owner's stripes
        self.parity = {}
        for owner, pidx, stripes in self._parity_batches():
            buf = np.zeros(len(stripes) * self.chunk_bytes, dtype=np.uint8)
            for n, s in enumerate(stripes):
                for pos, (r, c) in enumerate(s.data):
                    if r == self.rank:
                        buf[n * self.chunk_bytes:(n + 1) * self.chunk_bytes] = self._gfmul(int(self.G[pidx, pos]),
                                                                                           self._chunk(data, c))
            if owner is None:                       # host-only parity replicated on every member
                if self.world > 1:
                    t = torch.from_numpy(buf)
                    dist.all_reduce(t, op=dist.ReduceOp.BXOR, group=self.group)
                    buf = t.numpy()
                res = buf
            else:
                res = self._xor_reduce(buf, owner)
            if res is not None:
                for n, s in enumerate(stripes):
                    self.parity[(s.index, pidx)] = torch.from_numpy(
                        res[n * self.chunk_bytes:(n + 1) * self.chunk_bytes].copy())
        self.iteration = iteration
        t2 = time.perf_counter()
        self.stats = {"snapshot_s": t1 - t0, "encode_s": t2 - t1, "bytes": float(nbytes),
                      "encode_GBps": nbytes / max(t2 - t1, 1e-9) / 1e9}
        return self.stats

    def _parity_batches(self):
        """(owner group-rank or None, parity index, [stripes]) in an order every rank agrees on."""
        plan = self.plan
        if plan.stripes and plan.stripes[0].host_only:
            for i in range(self.m):
                yield None, i, plan.stripes
            return
        for owner in range(self.world):
            for i in range(self.m):
                ss = [s for s in plan.stripes if s.parity_owners[i] == owner]
                if ss:
                    yield owner, i, ss

    # ------------------------------------------------------------------ recover
    # -- state-dict form -------------------------------------------------------------------------------------------
    def save_state_dict(self, state_dict, iteration: int) -> Dict[str, float]:
        """Protect every tensor of a (nested, possibly sharded) state dict; its tensor-free structure is kept so
        that ``recover_state_dict`` can hand the same structure back."""
        from .tensor_aware import TensorAwareStateDict
        ta = TensorAwareStateDict.from_state_dict(state_dict, remove_redundant_data=False)
        tensors = ta.pop_tensors()
        self.hollow = ta
        return self.save(tensors, iteration)

    def recover_state_dict(self, lost_ranks: Sequence[int], hollow=None):
        """All ranks call.  Returns (iteration, state dict of this rank at that iteration).  A replacement rank has
        no structure of its own: it passes ``hollow``, a ``TensorAwareStateDict`` of a freshly built state dict
        (after ``pop_tensors``)."""
        ta = hollow if hollow is not None else getattr(self, "hollow", None)
        if ta is None:
            raise RuntimeError("no state-dict structure: pass hollow=TensorAwareStateDict.from_state_dict(...)")
        if not ta.is_hollow:
            ta.pop_tensors()
        ta.init_tensors()
        it = self.recover(lost_ranks, list(ta.tensors))
        self.hollow = ta
        return it, ta.to_state_dict()

    def drop_local_state(self) -> None:
        """Forget everything this rank holds (what a replacement process starts with)."""
        self.snapshot = None
        self.parity = {}

    def recover(self, lost_ranks: Sequence[int], tensors_out: Optional[Sequence[torch.Tensor]] = None) -> int:
        """Rebuild the saved bytes of every rank in ``lost_ranks`` (group ranks).  All ranks call.
        Returns the iteration of the recovered state; ``tensors_out`` (same shapes/dtypes as at
        save time) are overwritten with this rank's state at that iteration."""
        lost = sorted(set(int(r) for r in lost_ranks))
        if len(lost) > self.m:
            raise RuntimeError(f"{len(lost)} ranks lost but the code tolerates {self.m}")
        t0 = time.perf_counter()
        # agree on the iteration and the plan geometry (a replacement rank knows neither)
        meta = torch.tensor([self.iteration if self.iteration is not None else -1,
                             self.plan.chunks_per_rank if self.plan is not None else -1,
                             self.nbytes if self.rank not in lost else -1], dtype=torch.int64)
        sizes = None
        if self.world > 1:
            allm = [torch.zeros_like(meta) for _ in range(self.world)]
            dist.all_gather(allm, meta, group=self.group)
            it = max(int(a[0]) for a in allm)
            n_chunks = max(int(a[1]) for a in allm)
            sizes = [int(a[2]) for a in allm]
        else:
            it, n_chunks = int(meta[0]), int(meta[1])
        if it < 0:
            raise RuntimeError("no rank holds an in-memory checkpoint")
        self.iteration = it
        if self.plan is None or self.plan.chunks_per_rank != n_chunks:
            self.plan = plan_stripes(self.world, self.k, self.m, n_chunks)
        padded = n_chunks * self.chunk_bytes
        if self.rank in lost:
            self.snapshot = torch.zeros(padded, dtype=torch.uint8)
            self.parity = {}
        data = self.snapshot.numpy()
        k, m = self.k, self.m
        for s in self.plan.stripes:
            members: List[Tuple[str, int, int]] = [("d", r, c) for (r, c) in s.data]
            kk = len(members)
            lost_data = [pos for pos, (_, r, _) in enumerate(members) if r in lost]
            if s.host_only:
                lost_par: List[int] = []
            else:
                lost_par = [i for i, o in enumerate(s.parity_owners) if o in lost]
            if not lost_data and not lost_par:
                continue
            # member ids: 0..kk-1 data, k..k+m-1 parity (short stripes: absent data == zeros)
            present = [pos for pos in range(kk) if pos not in lost_data]
            present += [pos for pos in range(kk, k)]                    # virtual zero members
            if s.host_only:
                holder_of_par = {i: min(r for r in range(self.world) if r not in lost) for i in range(m)}
            else:
                holder_of_par = {i: o for i, o in enumerate(s.parity_owners) if o not in lost}
            present += [k + i for i in sorted(holder_of_par)]
            wanted = lost_data + [k + i for i in lost_par]
            M, use = gf256.decode_matrix(k, m, present, wanted)
            for w_i, w in enumerate(wanted):
                dst = members[w][1] if w < k else s.parity_owners[w - k]
                buf = np.zeros(self.chunk_bytes, dtype=np.uint8)
                for u_i, u in enumerate(use):
                    coef = int(M[w_i, u_i])
                    if coef == 0:
                        continue
                    if u < kk:
                        _, r, c = members[u]
                        if r == self.rank:
                            buf ^= self._gfmul(coef, self._chunk(data, c))
                    elif u >= k:
                        if holder_of_par[u - k] == self.rank:
                            buf ^= self._gfmul(coef, self.parity[(s.index, u - k)].numpy())
                res = self._xor_reduce(buf, dst)
                if res is not None:
                    if w < k:
                        self._chunk(data, members[w][2])[:] = res
                    else:
                        self.parity[(s.index, w - k)] = torch.from_numpy(res.copy())
        if self.rank in lost and sizes is not None and self.nbytes == 0 and tensors_out is not None:
            self.nbytes = sum(t.numel() * t.element_size() for t in tensors_out)
        if tensors_out is not None:
            o = 0
            for t in tensors_out:
                n = t.numel() * t.element_size()
                src = self.snapshot[o:o + n].view(t.dtype).view(t.shape)
                t.detach().copy_(src)
                o += n
        self.stats["recover_s"] = time.perf_counter() - t0
        return it
