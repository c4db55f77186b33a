"""Small tensor-parallel helpers (reference: megatron/core/tensor_parallel/utils.py:48-121)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from . import state


def divide(a: int, b: int) -> int:
    if a % b != 0:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


def split_tensor_along_last_dim(t: torch.Tensor, num_partitions: int, contiguous_split_chunks: bool = False):
    parts = torch.split(t, divide(t.shape[-1], num_partitions), dim=-1)
    return tuple(p.contiguous() for p in parts) if contiguous_split_chunks else parts


def split_tensor_into_1d_equal_chunks(t: torch.Tensor, new_buffer: bool = False) -> torch.Tensor:
    """This TP rank's 1/tp slice of the flattened tensor."""
    n = t.numel() // state.get_tensor_model_parallel_world_size()
    s = n * state.get_tensor_model_parallel_rank()
    flat = t.reshape(-1)[s:s + n]
    return flat.clone() if new_buffer else flat


def gather_split_1d_tensor(t: torch.Tensor) -> torch.Tensor:
    tp = state.get_tensor_model_parallel_world_size()
    out = torch.empty(t.numel() * tp, dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=state.get_tensor_model_parallel_group())
    return out


class VocabUtility:
    """[first, last) vocabulary range owned by a rank."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition: int, rank: int, world_size: int) -> Tuple[int, int]:
        return rank * per_partition, (rank + 1) * per_partition

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size: int, rank: int, world_size: int) -> Tuple[int, int]:
        return VocabUtility.vocab_range_from_per_partition_vocab_size(divide(global_vocab_size, world_size), rank,
                                                                      world_size)
