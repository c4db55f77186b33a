"""Partition-independent initialisation for parity tests: every parameter is drawn from a generator
seeded by its *global* name and then sliced for this rank, so TP/PP/VPP layouts of one model all
start from the same weights."""
import hashlib
import re

import torch

from megatron_lm_b200.parallel import state


def _seed(name: str) -> int:
    return int(hashlib.sha256(name.encode()).hexdigest()[:8], 16)


def reinit_by_global_name(module, config, std=0.05):
    tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
    tpr = state.get_tensor_model_parallel_rank() if state.model_parallel_is_initialized() else 0
    offset = getattr(getattr(module, "decoder", None), "layer_offset", 0)
    with torch.no_grad():
        for name, p in module.named_parameters():
            gname = re.sub(r"layers\.(\d+)\.", lambda m: f"layers.{int(m.group(1)) + offset}.", name)
            shape = list(p.shape)
            dim = getattr(p, "partition_dim", -1) if getattr(p, "tensor_model_parallel", False) else -1
            if dim >= 0 and tp > 1:
                shape[dim] *= tp
            g = torch.Generator().manual_seed(_seed(gname))
            if "layernorm" in gname and gname.endswith("weight"):
                full = 1.0 + 0.1 * torch.randn(shape, generator=g)
            else:
                full = std * torch.randn(shape, generator=g)
            if dim >= 0 and tp > 1:
                stride = getattr(p, "partition_stride", 1)
                per = p.shape[dim] // stride
                pieces = torch.split(full, per, dim=dim)
                full = torch.cat(pieces[tpr::tp], dim=dim)
            p.copy_(full.to(p.dtype))
