"""Batch plumbing: only TP rank 0 reads the data loader and broadcasts to its group; context-parallel
ranks then keep their two zig-zag sequence chunks (reference: megatron/training/utils.py:435-560,
megatron/core/utils.py:1833-1870, tensor_parallel/data.py:64)."""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..parallel import state


def _device():
    if torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def broadcast_data(keys, data: Optional[Dict[str, torch.Tensor]], datatype) -> Dict[str, torch.Tensor]:
    """Broadcast the tensors under ``keys`` from TP rank 0: sizes first, then one flat payload."""
    group = state.get_tensor_model_parallel_group()
    src = state.get_tensor_model_parallel_src_rank()
    if state.get_tensor_model_parallel_world_size() == 1:
        return {k: data[k].to(_device()) for k in keys}
    dev = _device()
    max_dim = 5
    sizes = torch.zeros(len(keys) * max_dim, dtype=torch.int64, device=dev)
    if state.get_tensor_model_parallel_rank() == 0:
        for i, k in enumerate(keys):
            for j, s in enumerate(data[k].shape):
                sizes[i * max_dim + j] = s
    dist.broadcast(sizes, src, group=group)
    shapes = []
    for i in range(len(keys)):
        sh = [int(x) for x in sizes[i * max_dim:(i + 1) * max_dim].tolist() if x > 0]
        shapes.append(sh)
    total = sum(int(torch.tensor(s).prod()) for s in shapes)
    if state.get_tensor_model_parallel_rank() == 0:
        flat = torch.cat([data[k].reshape(-1).to(datatype) for k in keys]).to(dev)
    else:
        flat = torch.empty(total, dtype=datatype, device=dev)
    dist.broadcast(flat, src, group=group)
    out, o = {}, 0
    for k, sh in zip(keys, shapes):
        n = int(torch.tensor(sh).prod())
        out[k] = flat[o:o + n].view(*sh)
        o += n
    return out


def get_batch_on_this_tp_rank(data_iterator, args) -> Dict[str, torch.Tensor]:
    data = None
    if state.get_tensor_model_parallel_rank() == 0:
        data = next(data_iterator)
    ints = broadcast_data(["tokens", "labels", "position_ids"], data, torch.int64)
    floats = broadcast_data(["loss_mask"], data, torch.float32)
    out = {**ints, **floats}
    if getattr(args, "create_attention_mask_in_dataloader", False) and (data is None or "attention_mask" in data):
        out.update(broadcast_data(["attention_mask"], data, torch.bool))
    return out


def get_batch_on_this_cp_rank(batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Keep sequence chunks r and 2cp-1-r of 2cp equal chunks (balanced causal work)."""
    cp = state.get_context_parallel_world_size()
    if cp == 1:
        return batch
    r = state.get_context_parallel_rank()
    out = {}
    for k, v in batch.items():
        if v is None:
            out[k] = v
            continue
        dim = 2 if k == "attention_mask" else 1
        shape = list(v.shape)
        v2 = v.view(*shape[:dim], 2 * cp, shape[dim] // (2 * cp), *shape[dim + 1:])
        idx = torch.tensor([r, 2 * cp - 1 - r], device=v.device)
        v2 = v2.index_select(dim, idx)
        out[k] = v2.reshape(*shape[:dim], -1, *shape[dim + 1:])
    return out
