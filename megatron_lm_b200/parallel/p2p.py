"""Pipeline point-to-point transfers over the pipeline group (NCCL on GPUs, Gloo on CPU).

The reference exposes nine send/recv combinations built on ``batch_isend_irecv``
(megatron/core/pipeline_parallel/p2p_communication.py:119-604).  Here a
communicator object owns the fixed activation shape and dtype of the run and
offers four primitives - post a receive from the previous / next stage, send to
the next / previous stage - all non-blocking; the schedule executor decides when
to wait.  Sends are kept alive until complete and drained at the end of the step.
Variable sequence lengths exchange a 3-element shape tensor first (:21).

Each of the four message streams of a stage (activations in from the previous stage, activations out to the next,
gradients in from the next, gradients out to the previous) runs on a communicator of its own
(``state.get_pipeline_channel``), so every communicator is a one-way FIFO.  The reference instead batches the sends
and receives of one schedule step into one NCCL group (``batch_isend_irecv``); un-batched transfers of both
directions on one communicator can block each other, because NCCL runs them in issue order on one stream.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import state


class _Pending:
    __slots__ = ("tensor", "work")

    def __init__(self, tensor, work):
        self.tensor, self.work = tensor, work


class P2PCommunicator:
    def __init__(self, group, pp_rank: int, pp_size: int, shape: Tuple[int, ...], dtype, config=None):
        self.group, self.rank, self.size = group, pp_rank, pp_size
        self.shape, self.dtype = tuple(shape), dtype
        self.config = config
        self.variable = bool(config.variable_seq_lengths) if config is not None else False
        self.prev = dist.get_global_rank(group, (pp_rank - 1) % pp_size) if group is not None else None
        self.next = dist.get_global_rank(group, (pp_rank + 1) % pp_size) if group is not None else None
        self._sends: List[_Pending] = []
        backend = dist.get_backend(group) if group is not None else "gloo"
        self.device = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
        prev_stage = (pp_rank - 1) % pp_size

        def channel(kind, sender_stage):
            ch = state.get_pipeline_channel(kind, sender_stage) if state.model_parallel_is_initialized() else None
            return ch if ch is not None else group
        self.ch_fwd_out = channel("F", pp_rank)        # activations to the next stage
        self.ch_fwd_in = channel("F", prev_stage)      # activations from the previous stage
        self.ch_bwd_in = channel("B", pp_rank)         # gradients from the next stage
        self.ch_bwd_out = channel("B", prev_stage)     # gradients to the previous stage

    # -- receives ------------------------------------------------------------
    def _irecv(self, src: int, ch) -> _Pending:
        shape = self.shape
        if self.variable:
            sh = torch.empty(3, dtype=torch.int64, device=self.device)
            dist.recv(sh, src=src, group=ch)
            shape = tuple(int(x) for x in sh.tolist())
        buf = torch.empty(shape, dtype=self.dtype, device=self.device)
        return _Pending(buf, dist.irecv(buf, src=src, group=ch))

    def irecv_forward(self) -> _Pending:
        """Activation from the previous stage (the last stage's sender for rank 0 of a later chunk)."""
        return self._irecv(self.prev, self.ch_fwd_in)

    def irecv_backward(self) -> _Pending:
        """Output gradient from the next stage."""
        return self._irecv(self.next, self.ch_bwd_in)

    def wait(self, pending: Optional[_Pending]) -> Optional[torch.Tensor]:
        if pending is None:
            return None
        pending.work.wait()
        return pending.tensor

    # -- sends -----------------------------------------------------------------
    def _isend(self, t: torch.Tensor, dst: int, ch) -> None:
        t = t.detach().contiguous()
        if t.dtype != self.dtype:
            t = t.to(self.dtype)
        if self.variable:
            sh = torch.tensor(list(t.shape) + [1] * (3 - t.dim()), dtype=torch.int64, device=self.device)
            dist.send(sh, dst=dst, group=ch)
        self._sends.append(_Pending(t, dist.isend(t, dst=dst, group=ch)))
        self._reap()

    def send_forward(self, t: torch.Tensor) -> None:
        self._isend(t, self.next, self.ch_fwd_out)

    def send_backward(self, t: torch.Tensor) -> None:
        self._isend(t, self.prev, self.ch_bwd_out)

    def warmup(self) -> None:
        """One tiny message over each channel, so the communicators exist before the first timed or
        latency-sensitive step (NCCL builds a communicator at its first use, which can take seconds)."""
        one = torch.ones(1, dtype=torch.float32, device=self.device)
        prev_stage = (self.rank - 1) % self.size
        # every rank touches its channels in one global order, (kind, sender stage): a communicator that is built
        # at first use blocks the host until both members arrive, and a common order rules out a cycle of waits
        mine = {("F", self.rank): ("send", self.next, self.ch_fwd_out), ("F", prev_stage): ("recv", self.prev, self.ch_fwd_in),
                ("B", self.rank): ("recv", self.next, self.ch_bwd_in), ("B", prev_stage): ("send", self.prev, self.ch_bwd_out)}
        works, keep = [], []
        for key in sorted(mine):
            op, peer, ch = mine[key]
            if op == "send":
                works.append(dist.isend(one, dst=peer, group=ch))
            else:
                buf = torch.empty_like(one)
                keep.append(buf)
                works.append(dist.irecv(buf, src=peer, group=ch))
        for w in works:
            w.wait()
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    def _reap(self) -> None:
        self._sends = [p for p in self._sends if not p.work.is_completed()]

    def drain(self) -> None:
        for p in self._sends:
            p.work.wait()
        self._sends = []
