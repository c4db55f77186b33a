"""GPU energy accounting through NVML's total-energy counter (reference:
megatron/core/energy_monitor.py:22-91).  Read-only: no clock, power-limit or mode is ever set."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class EnergyMonitor:
    def __init__(self, nvml=None, device_index: Optional[int] = None):
        self._nvml = nvml
        self._handle = None
        self._total = 0.0
        self._lap = 0.0
        self._last = None
        self._paused = True
        self._dev = device_index

    def setup(self):
        if self._nvml is None:
            import pynvml
            self._nvml = pynvml
        self._nvml.nvmlInit()
        idx = self._dev if self._dev is not None else (torch.cuda.current_device() if torch.cuda.is_available() else 0)
        self._handle = self._nvml.nvmlDeviceGetHandleByIndex(idx)

    def _read_j(self) -> float:
        return self._nvml.nvmlDeviceGetTotalEnergyConsumption(self._handle) / 1000.0      # mJ -> J

    def resume(self):
        self._last = self._read_j()
        self._paused = False

    def pause(self):
        if not self._paused:
            self._tick()
            self._paused = True

    def _tick(self):
        now = self._read_j()
        self._total += now - self._last
        self._lap += now - self._last
        self._last = now

    def lap(self) -> float:
        """Joules (summed over ranks) since the previous lap."""
        if not self._paused:
            self._tick()
        e, self._lap = self._lap, 0.0
        if dist.is_initialized() and dist.get_world_size() > 1:
            dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
            t = torch.tensor([e], dtype=torch.float64, device=dev)
            dist.all_reduce(t)
            e = float(t.item())
        return e

    def get_total(self) -> float:
        if not self._paused:
            self._tick()
        return self._total

    def shutdown(self):
        if self._nvml is not None:
            self._nvml.nvmlShutdown()
