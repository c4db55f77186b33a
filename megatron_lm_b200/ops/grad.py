"""How parameter gradients leave an op.

Parameters owned by a gradient buffer carry ``main_grad`` (a view into the flat
fp32/bf16 buffer) and, optionally, ``grad_ready`` - a callable the owning bucket
installs.  Ops of this library accumulate straight into ``main_grad`` (the
reference does this only for linear weights, through an Apex kernel:
megatron/core/tensor_parallel/layers.py:553-598) and then signal readiness, so
no autograd hook and no temporary ``.grad`` tensor is involved.
"""
from __future__ import annotations

from typing import Optional

import torch


def has_main_grad(p: Optional[torch.Tensor]) -> bool:
    return p is not None and getattr(p, "main_grad", None) is not None


def notify_ready(p: torch.Tensor) -> None:
    cb = getattr(p, "grad_ready", None)
    if cb is not None:
        cb()


def deliver(p: torch.Tensor, g: torch.Tensor) -> Optional[torch.Tensor]:
    """Add ``g`` into ``p.main_grad`` when there is one (returns None), else
    return ``g`` in the parameter's dtype for autograd to accumulate."""
    if has_main_grad(p):
        mg = p.main_grad
        if g.is_cuda:
            from . import _lib
            g = g.contiguous()
            _lib.check(_lib.lib().mlb_cast(_lib.dt(g), _lib.dt(mg), g.data_ptr(), mg.data_ptr(), g.numel(), 1.0, 1,
                                           _lib.stream()), "grad accumulate")
        else:
            mg.add_(g.to(mg.dtype).view_as(mg))
        notify_ready(p)
        return None
    return g.to(p.dtype).view_as(p)
