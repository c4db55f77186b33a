"""Restart a training function inside the same processes after a rank-local failure.

Reference: megatron/training/inprocess_restart.py (``inprocess_restart`` :19, ``maybe_wrap_for_inprocess_restart``
:119) builds on an external in-process restart library (rank health monitoring, collective abort, re-rendezvous).
Here the same contract is implemented on a TCP store:

* every rank runs ``fn(attempt, store)`` inside ``RestartWrapper``;
* a rank whose attempt raises publishes the failure under the attempt's key; healthy ranks notice it either
  between steps (``wrapper.check()``) or when their next collective fails, and raise ``RestartSignal``;
* all ranks tear down the process groups of the attempt, meet at a store barrier, and run the next attempt
  with a fresh store prefix, up to ``max_restarts`` times.

Failures are host-side events only (an exception, a rank that never arrives); nothing here touches a GPU.
"""
from __future__ import annotations

import time
import traceback
from typing import Callable, Optional

import torch.distributed as dist


class RestartSignal(RuntimeError):
    """Raised on healthy ranks to abandon the current attempt."""


class RestartWrapper:
    def __init__(self, store, rank: int, world_size: int, max_restarts: int = 3, barrier_timeout: float = 60.0,
                 finalize: Optional[Callable[[], None]] = None):
        self.store, self.rank, self.world = store, rank, world_size
        self.max_restarts, self.barrier_timeout = max_restarts, barrier_timeout
        self.finalize = finalize
        self.attempt = 0

    # -- called from inside fn ----------------------------------------------------------
    def _key(self, what: str) -> str:
        return f"inprocess/{self.attempt}/{what}"

    def check(self) -> None:
        """Between steps: leave the attempt if any rank has failed."""
        if self.store.num_keys() and self._failed():
            raise RestartSignal(f"another rank failed in attempt {self.attempt}")

    def step_barrier(self, step: int, poll_s: float = 0.002) -> None:
        """Between steps: wait until every rank has finished ``step`` or some rank has failed.  Unlike ``check``
        this cannot miss a failure that is published a moment later - the failed rank never arrives, so the
        healthy ranks are still here when its flag appears - at the price of one store round trip per step."""
        key = self._key(f"step{step}")
        self.store.add(key, 1)
        t0 = time.time()
        while int(self.store.add(key, 0)) < self.world:
            if self._failed():
                raise RestartSignal(f"another rank failed in attempt {self.attempt} (seen at step {step})")
            if time.time() - t0 > self.barrier_timeout:
                raise TimeoutError(f"rank {self.rank}: step barrier {step} of attempt {self.attempt} timed out")
            time.sleep(poll_s)

    def _failed(self) -> bool:
        try:
            return int(self.store.add(self._key("failed"), 0)) > 0
        except Exception:
            return False

    # -- driver ---------------------------------------------------------------------------
    def _barrier(self, name: str) -> None:
        key = self._key(name)
        self.store.add(key, 1)
        t0 = time.time()
        while int(self.store.add(key, 0)) < self.world:
            if time.time() - t0 > self.barrier_timeout:
                raise TimeoutError(f"rank {self.rank}: barrier {name} of attempt {self.attempt} timed out")
            time.sleep(0.01)

    def run(self, fn: Callable):
        last_error = None
        while self.attempt <= self.max_restarts:
            try:
                out = fn(self, self.attempt)
                # nobody may return while another rank is about to ask for a restart
                self._barrier("done")
                if self._failed():
                    raise RestartSignal("a rank failed after this rank finished")
                return out
            except BaseException as e:              # noqa: BLE001 - every failure is a reason to restart
                if isinstance(e, (KeyboardInterrupt, SystemExit)):
                    raise
                if not isinstance(e, RestartSignal):
                    last_error = traceback.format_exc()
                    print(f"[rank {self.rank}] attempt {self.attempt} failed; asking every rank to restart\n"
                          f"{last_error}", flush=True)
                    try:
                        self.store.add(self._key("failed"), 1)
                    except Exception:
                        pass
                if self.finalize is not None:
                    try:
                        self.finalize()
                    except Exception:
                        pass
                if dist.is_initialized():
                    try:
                        dist.destroy_process_group()
                    except Exception:
                        pass
                self._barrier("restart")
                self.attempt += 1
        raise RuntimeError(f"rank {self.rank}: giving up after {self.max_restarts} restarts\n{last_error or ''}")


def maybe_wrap_for_inprocess_restart(pretrain_fn: Callable, args=None):
    """Returns (function to call, store or None): wraps ``pretrain_fn`` when ``--inprocess-restart`` is set."""
    if args is None or not getattr(args, "inprocess_restart", False):
        return pretrain_fn, None
    import os
    from datetime import timedelta
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    port = int(os.environ.get("MASTER_PORT", 29500)) + 1
    store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), port, world, is_master=(rank == 0),
                          timeout=timedelta(seconds=300), wait_for_workers=True)
    wrapper = RestartWrapper(store, rank, world, max_restarts=getattr(args, "inprocess_max_iterations", None) or 3,
                             barrier_timeout=float(getattr(args, "inprocess_barrier_timeout", None) or 120.0))

    def wrapped(*a, **kw):
        return wrapper.run(lambda w, attempt: pretrain_fn(*a, inprocess_call_wrapper=w, **kw))
    return wrapped, store
