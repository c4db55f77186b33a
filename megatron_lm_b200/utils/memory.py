"""Named, reusable scratch tensors (reference: megatron/core/utils.py:500
``GlobalMemoryBuffer``).  A buffer is grown on demand and handed out as a view,
so per-step workspaces (sequence-parallel gather targets, reduction partials)
cost no allocator traffic in the steady state."""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch


class GlobalMemoryBuffer:
    def __init__(self):
        self.buffer: Dict[Tuple[str, torch.dtype, str], torch.Tensor] = {}

    def get_tensor(self, tensor_shape, dtype, name, device=None) -> torch.Tensor:
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        device = torch.device(device)
        need = int(math.prod(tensor_shape))
        key = (name, dtype, str(device))
        buf = self.buffer.get(key)
        if buf is None or buf.numel() < need:
            buf = torch.empty(max(need, 1), dtype=dtype, device=device, requires_grad=False)
            self.buffer[key] = buf
        return buf[:need].view(*tensor_shape)


_workspace = GlobalMemoryBuffer()


def workspace(shape, dtype, name, device=None) -> torch.Tensor:
    """Process-wide scratch used by kernels that need partial-sum space."""
    return _workspace.get_tensor(shape, dtype, name, device)
