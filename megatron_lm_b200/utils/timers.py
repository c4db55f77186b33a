"""Named timers with cross-rank reporting (reference: megatron/core/timers.py:96-452).

Timers use CUDA events on the current stream when a GPU is present, so starting and stopping one
never forces a device synchronisation on the hot path; elapsed times are resolved lazily when
they are read (the reference synchronises the device at every start/stop)."""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class Timer:
    def __init__(self, name: str, use_cuda: Optional[bool] = None):
        self.name = name
        self.cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self._elapsed = 0.0
        self._active_time = 0.0
        self._pending: List = []
        self._started = False
        self._t0 = None
        self._barrier_group = None

    def set_barrier_group(self, group):
        self._barrier_group = group

    def start(self, barrier: bool = False):
        if self._started:
            raise RuntimeError(f"timer {self.name} has already been started")
        if barrier and dist.is_initialized():
            dist.barrier(group=self._barrier_group)
        if self.cuda:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        else:
            self._t0 = time.perf_counter()
        self._started = True

    def stop(self, barrier: bool = False):
        if not self._started:
            raise RuntimeError(f"timer {self.name} is not started")
        if barrier and dist.is_initialized():
            dist.barrier(group=self._barrier_group)
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pending.append((self._t0, e))
        else:
            dt = time.perf_counter() - self._t0
            self._elapsed += dt
            self._active_time += dt
        self._started = False

    def _resolve(self):
        for a, b in self._pending:
            b.synchronize()
            dt = a.elapsed_time(b) / 1e3
            self._elapsed += dt
            self._active_time += dt
        self._pending = []

    def reset(self):
        self._resolve()
        self._elapsed = 0.0
        self._started = False

    def elapsed(self, reset: bool = True, barrier: bool = False) -> float:
        was = self._started
        if was:
            self.stop(barrier=barrier)
        self._resolve()
        out = self._elapsed
        if reset:
            self._elapsed = 0.0
        if was:
            self.start(barrier=barrier)
        return out

    def active_time(self) -> float:
        self._resolve()
        return self._active_time


class _Dummy:
    def start(self, barrier=False): pass
    def stop(self, barrier=False): pass
    def reset(self): pass
    def elapsed(self, reset=True, barrier=False): return 0.0
    def active_time(self): return 0.0


class Timers:
    """``timers(name, log_level)`` returns a live timer when ``log_level`` <= the configured level,
    else a no-op.  ``log_option`` is one of max / minmax / all."""

    def __init__(self, log_level: int = 0, log_option: str = "minmax"):
        self._log_level, self._log_option = log_level, log_option
        self._timers: Dict[str, Timer] = {}
        self._levels: Dict[str, int] = {}
        self._dummy = _Dummy()
        self._max_log_level = 2

    def __call__(self, name: str, log_level: Optional[int] = None):
        if name in self._timers:
            if log_level is not None and log_level != self._levels[name]:
                raise ValueError(f"timer {name} was created with log level {self._levels[name]}")
            return self._timers[name]
        log_level = self._max_log_level if log_level is None else log_level
        if log_level > self._max_log_level:
            raise ValueError("log level above the maximum")
        if log_level > self._log_level:
            return self._dummy
        self._timers[name] = Timer(name)
        self._levels[name] = log_level
        return self._timers[name]

    def _gather(self, names, reset, barrier):
        """[world, len(names)] elapsed seconds (one all-gather)."""
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        local = torch.tensor([self._timers[n].elapsed(reset=reset) if n in self._timers else 0.0 for n in names],
                             dtype=torch.float32)
        if world == 1:
            return local.view(1, -1)
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        buf = torch.zeros(world, len(names), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(buf.view(-1), local.to(dev))
        return buf.cpu()

    def get_all_timers_string(self, names=None, normalizer: float = 1.0, reset: bool = True, barrier: bool = False):
        names = list(self._timers.keys()) if names is None else [n for n in names if n in self._timers]
        if not names:
            return None
        t = self._gather(names, reset, barrier) / normalizer * 1000.0
        lines = []
        if self._log_option in ("max", "minmax"):
            lines.append("(min, max) time across ranks (ms):" if self._log_option == "minmax" else
                         "max time across ranks (ms):")
            for i, n in enumerate(names):
                col = t[:, i]
                if col.max() <= 0:
                    continue
                if self._log_option == "minmax":
                    lines.append(f"    {n:.<48}: ({col[col > 0].min():.2f}, {col.max():.2f})")
                else:
                    lines.append(f"    {n:.<48}: {col.max():.2f}")
        else:
            lines.append("times across ranks (ms):")
            for i, n in enumerate(names):
                lines.append(f"  {n}:")
                for r in range(t.shape[0]):
                    lines.append(f"     rank {r:2d}: {t[r, i]:.2f}")
        if len(lines) <= 1:
            return None                      # nothing was timed since the last report: no bare heading
        return "\n".join(lines)

    def log(self, names=None, rank=None, normalizer: float = 1.0, reset: bool = True, barrier: bool = False):
        s = self.get_all_timers_string(names, normalizer, reset, barrier)
        me = dist.get_rank() if dist.is_initialized() else 0
        if rank is None:
            rank = (dist.get_world_size() - 1) if dist.is_initialized() else 0
        if s is not None and me == rank:
            print(s, flush=True)

    def write(self, names, writer, iteration: int, normalizer: float = 1.0, reset: bool = True, barrier: bool = False):
        # every rank takes part in the gather (a collective); only the rank that holds a writer records the result.
        # The name list must therefore be the same on all ranks: timers a rank never started count as zero.
        names = list(names)
        if not names:
            return
        t = self._gather(names, reset, barrier) / normalizer
        if writer is None:
            return
        for i, n in enumerate(names):
            writer.add_scalar(n + "-time", float(t[:, i].max()), iteration)
