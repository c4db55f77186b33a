"""Dense -> mixture-of-experts upcycling of model weights.

Reference: megatron/core/transformer/moe/upcycling_utils.py (``upcycle_state_dict`` :232,
granular upcycling :94-190).  Every expert starts as a copy of the dense MLP; the router starts
from small random values (or zeros); with ``granularity`` g > 1 each expert takes a 1/g slice of the
dense FFN (and the expert count must be a multiple of g), scaling fc2 so that the top-k mixture
reproduces the dense output at initialisation.
"""
from __future__ import annotations

import re
from typing import Dict

import torch


def upcycle_state_dict(dense_sd: Dict[str, torch.Tensor], num_experts: int, moe_layers=None, granularity: int = 1,
                       gated: bool = True, router_std: float = 0.02, topk: int = 2, seed: int = 0):
    """Keys ``decoder.layers.N.mlp.linear_fc{1,2}.weight`` of the layers in ``moe_layers`` (default all) become
    ``mlp.experts.weight{1,2}`` [E, ...] and a router weight ``mlp.router.weight`` [E, h] is added."""
    out = {}
    g = torch.Generator().manual_seed(seed)
    if num_experts % granularity:
        raise ValueError("num_experts must be a multiple of the granularity")
    for k, v in dense_sd.items():
        m = re.match(r"^(.*decoder\.layers\.(\d+)\.mlp\.)linear_fc([12])\.weight$", k)
        if not m or (moe_layers is not None and int(m.group(2)) not in moe_layers):
            out[k] = v
            continue
        prefix, which = m.group(1), m.group(3)
        if which == "1":
            if granularity > 1:
                parts = (v.chunk(2, 0) if gated else (v,))
                slices = [torch.cat([p.chunk(granularity, 0)[j] for p in parts], 0) for j in range(granularity)]
                w = torch.stack([slices[e % granularity] for e in range(num_experts)])
            else:
                w = v.unsqueeze(0).repeat(num_experts, 1, 1)
            out[prefix + "experts.weight1"] = w.clone()
            h = v.shape[1]
            out[prefix + "router.weight"] = torch.randn(num_experts, h, generator=g, dtype=torch.float32).to(v.dtype) * router_std
        else:
            if granularity > 1:
                slices = v.chunk(granularity, 1)
                w = torch.stack([slices[e % granularity] for e in range(num_experts)]) * (granularity / topk * 1.0)
            else:
                w = v.unsqueeze(0).repeat(num_experts, 1, 1)
            out[prefix + "experts.weight2"] = w.clone()
    return out
