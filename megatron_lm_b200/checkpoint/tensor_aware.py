"""A state dict that knows which of its leaves are tensors: the bridge between a (sharded) state dict and the
in-memory checkpoint tiers, which move flat lists of tensors.

``TensorAwareStateDict.from_state_dict(sd)`` records the nested structure once.  ``pop_tensors()`` hands the tensors
out (leaving a *hollow* structure that is cheap to pickle, send to a peer or keep on the host), ``insert_tensors()``
puts tensors of the same shapes back, ``copy_tensors_to_cpu`` / ``restore_tensor_device`` move a snapshot between
devices, ``to_state_dict()`` rebuilds the ordinary state dict.  With ``ShardedTensor`` leaves only the main replicas
carry data (``remove_redundant_data``), as each tensor needs protecting once per job.

Reference: megatron/core/dist_checkpointing/tensor_aware_state_dict.py:48-340 (``MCoreTensorAwareStateDict`` for
local checkpoints: ``from_state_dict`` :101, ``is_hollow`` :155, ``pop_tensors`` :193, ``insert_tensors`` :213,
``init_tensors`` :230, ``copy_tensors_to_cpu`` :245, ``restore_tensor_device`` :264, ``to_state_dict`` :325).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Iterable, Iterator, List, Optional, Tuple

import torch

from .sharded import ShardedTensor


@dataclass
class _Slot:
    """Where a tensor sits in the structure and what it looks like."""
    path: Tuple
    shape: Tuple[int, ...]
    dtype: torch.dtype
    device: torch.device
    sharded: bool


class TensorAwareStateDict:
    def __init__(self, structure: Any, slots: List[_Slot], tensors: Optional[List[torch.Tensor]]):
        self._structure, self._slots, self._tensors = structure, slots, tensors
        self._orig_devices = [s.device for s in slots]

    # -- construction ---------------------------------------------------------------------------------------------
    @classmethod
    def from_state_dict(cls, state_dict: Any, remove_redundant_data: bool = True) -> "TensorAwareStateDict":
        """Walks dicts / lists / tuples.  Tensor leaves and the data of ``ShardedTensor`` leaves are taken out of the
        structure (it keeps a placeholder).  With ``remove_redundant_data`` a ShardedTensor that is not the main
        replica is recorded without data: another rank protects it."""
        slots: List[_Slot] = []
        tensors: List[torch.Tensor] = []

        def walk(x, path):
            if isinstance(x, torch.Tensor):
                slots.append(_Slot(path, tuple(x.shape), x.dtype, x.device, False))
                tensors.append(x)
                return _Hole(len(slots) - 1)
            if isinstance(x, ShardedTensor):
                meta = ShardedTensor(x.key, None, x.dtype, x.local_shape, x.global_shape, x.global_offset,
                                     x.axis_fragmentations, x.replica_id, x.prepend_axis_num, x.allow_shape_mismatch,
                                     x.flattened_range)
                if x.data is None or (remove_redundant_data and not x.is_main_replica()):
                    return meta
                slots.append(_Slot(path, tuple(x.data.shape), x.data.dtype, x.data.device, True))
                tensors.append(x.data)
                return _ShardedHole(len(slots) - 1, meta)
            if isinstance(x, dict):
                return {k: walk(v, path + (k,)) for k, v in x.items()}
            if isinstance(x, (list, tuple)):
                out = [walk(v, path + (i,)) for i, v in enumerate(x)]
                return out if isinstance(x, list) else tuple(out)
            return x
        return cls(walk(state_dict, ()), slots, tensors)

    # -- tensors --------------------------------------------------------------------------------------------------
    @property
    def is_hollow(self) -> bool:
        return self._tensors is None

    @property
    def tensors(self) -> Iterator[torch.Tensor]:
        if self.is_hollow:
            raise RuntimeError("the tensors were popped: insert_tensors() or init_tensors() first")
        return iter(self._tensors)

    @property
    def common_state_dict(self) -> Any:
        """The structure without any tensor data (placeholders where tensors go)."""
        return self._structure

    def nbytes(self) -> int:
        n = 0
        for s in self._slots:
            k = 1
            for d in s.shape:
                k *= d
            n += k * torch.empty((), dtype=s.dtype).element_size()
        return n

    def pop_tensors(self) -> List[torch.Tensor]:
        if self.is_hollow:
            raise RuntimeError("already hollow")
        out, self._tensors = self._tensors, None
        return out

    def insert_tensors(self, tensor_data: Iterable[torch.Tensor]) -> None:
        if not self.is_hollow:
            raise RuntimeError("the state dict still holds its tensors")
        data = list(tensor_data)
        if len(data) != len(self._slots):
            raise ValueError(f"{len(data)} tensors for {len(self._slots)} places")
        for t, s in zip(data, self._slots):
            if tuple(t.shape) != s.shape or t.dtype != s.dtype:
                raise ValueError(f"tensor for {'.'.join(map(str, s.path))}: {tuple(t.shape)} {t.dtype}, "
                                 f"expected {s.shape} {s.dtype}")
        self._tensors = data

    def init_tensors(self) -> None:
        """Empty tensors of the recorded shapes on the recorded devices (a receive buffer for a peer's copy)."""
        self.insert_tensors([torch.empty(s.shape, dtype=s.dtype, device=d) for s, d in zip(self._slots, self._orig_devices)])

    def copy_tensors_to_cpu(self, non_blocking: bool = False) -> None:
        """Replace every tensor by a host copy (pinned when a GPU is present, so the copy can run asynchronously)."""
        pin = torch.cuda.is_available()
        out = []
        for t in self.tensors:
            if t.device.type == "cpu":
                out.append(t.detach().clone())
                continue
            h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=pin)
            h.copy_(t.detach(), non_blocking=non_blocking)
            out.append(h)
        self._tensors = out

    def restore_tensor_device(self, non_blocking: bool = True) -> None:
        """Move every tensor back to the device it was on when the structure was recorded."""
        self._tensors = [t.to(d, non_blocking=non_blocking) if t.device != d else t
                         for t, d in zip(self.tensors, self._orig_devices)]

    # -- back to an ordinary state dict -------------------------------------------------------------------------------
    def to_state_dict(self) -> Any:
        if self.is_hollow:
            raise RuntimeError("hollow: nothing to rebuild from")
        ts = self._tensors

        def build(x):
            if isinstance(x, _Hole):
                return ts[x.index]
            if isinstance(x, _ShardedHole):
                m = x.meta
                return ShardedTensor(m.key, ts[x.index], m.dtype, m.local_shape, m.global_shape, m.global_offset,
                                     m.axis_fragmentations, m.replica_id, m.prepend_axis_num, m.allow_shape_mismatch,
                                     m.flattened_range)
            if isinstance(x, dict):
                return {k: build(v) for k, v in x.items()}
            if isinstance(x, list):
                return [build(v) for v in x]
            if isinstance(x, tuple):
                return tuple(build(v) for v in x)
            return x
        return build(self._structure)


@dataclass(frozen=True)
class _Hole:
    index: int


@dataclass(frozen=True)
class _ShardedHole:
    index: int
    meta: ShardedTensor
