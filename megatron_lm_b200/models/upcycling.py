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


# ------------------------------------------------------------------------------------------------ live models
def _dense_name(moe_key: str):
    """MoE parameter name -> (dense parameter name, which, expert index or None)."""
    m = re.match(r"^(.*\.mlp\.)experts\.weight([12])$", moe_key)
    if m:
        return f"{m.group(1)}linear_fc{m.group(2)}.weight", m.group(2), None
    m = re.match(r"^(.*\.mlp\.)experts\.local_experts\.(\d+)\.linear_fc([12])\.(weight|bias)$", moe_key)
    if m:
        return f"{m.group(1)}linear_fc{m.group(3)}.{m.group(4)}", m.group(3), int(m.group(2))
    return None, None, None


@torch.no_grad()
def upcycle_model(dense_model, moe_model, granularity: int = 1, router_std: float = 0.02, seed: int = 1234) -> Dict[str, str]:
    """Fill ``moe_model`` from ``dense_model`` (same depth, width, attention; this rank's shards of both):
    everything the two share is copied, every local expert becomes a copy of the dense MLP of its layer (a 1/g slice
    of it with ``granularity`` g, second projection rescaled so that the top-k mixture reproduces the dense output),
    routers draw small normal values from a generator seeded alike on every rank.  Returns {moe name: source}.
    Reference: megatron/core/transformer/moe/upcycling_utils.py:108-330 (``_convert_to_moe_state_dict``,
    ``upcycle_state_dict``, ``load_and_upcycle_model``)."""
    cfg = moe_model.config
    dense_sd = dict(dense_model.state_dict())
    gated = cfg.gated_linear_unit
    E = cfg.num_moe_experts
    topk = cfg.moe_router_topk
    if E % granularity:
        raise ValueError("the number of experts must be a multiple of the upcycling granularity")
    report: Dict[str, str] = {}
    gen = torch.Generator().manual_seed(seed)

    def expert_slice(w, which, e_global):
        if granularity == 1:
            return w
        j = e_global % granularity
        if which == "1":
            parts = w.chunk(2, 0) if gated else (w,)
            return torch.cat([p.chunk(granularity, 0)[j] for p in parts], 0)
        return w.chunk(granularity, 1)[j] * (granularity / topk)

    ep_rank = 0
    try:
        from ..parallel import state
        if state.model_parallel_is_initialized():
            ep_rank = state.get_expert_model_parallel_rank()
    except Exception:
        pass
    for name, p in moe_model.named_parameters():
        dense_key, which, e_local = _dense_name(name)
        if name in dense_sd and dense_sd[name].shape == p.shape:
            p.copy_(dense_sd[name])
            report[name] = "copied"
        elif dense_key is not None and dense_key in dense_sd:
            w = dense_sd[dense_key]
            if w.dim() == 1:                                           # a bias of a per-expert MLP
                p.copy_(w if which == "2" or granularity == 1 else expert_slice(w.unsqueeze(1), "1", e_local).squeeze(1))
                report[name] = f"{dense_key}"
                continue
            if e_local is None:                                        # grouped experts: [local E, out, in]
                n_local = p.shape[0]
                for e in range(n_local):
                    src = expert_slice(w, which, ep_rank * n_local + e)
                    if src.shape != p[e].shape:
                        raise ValueError(f"{name}: expert shape {tuple(p[e].shape)} does not match the dense MLP's "
                                         f"{tuple(src.shape)} (tensor-parallel sizes of experts and dense layers differ?)")
                    p[e].copy_(src)
            else:
                n_local = E // max(1, _ep_size())
                src = expert_slice(w, which, ep_rank * n_local + e_local)
                if src.shape != p.shape:
                    raise ValueError(f"{name}: shape {tuple(p.shape)} does not match the dense MLP's {tuple(src.shape)}")
                p.copy_(src)
            report[name] = f"{dense_key}"
        elif name.endswith("mlp.router.weight"):
            p.copy_((torch.randn(p.shape, generator=gen, dtype=torch.float32) * router_std).to(p.dtype))
            report[name] = "router init"
        else:
            report[name] = "kept"
    return report


def _ep_size() -> int:
    try:
        from ..parallel import state
        return state.get_expert_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
    except Exception:
        return 1


def dense_args_for_upcycling(args):
    """The arguments of the dense model a mixture-of-experts run is upcycled from: no experts, the dense FFN width
    (``--ffn-hidden-size``; with granularity g the experts' width is 1/g of it)."""
    import copy
    d = copy.copy(args)
    d.num_experts = None
    d.moe_ffn_hidden_size = None
    d.expert_model_parallel_size = 1
    d.moe_shared_expert_intermediate_size = None
    d.moe_layer_freq = 1
    return d
