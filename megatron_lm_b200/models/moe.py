"""Mixture-of-experts layer: router, token dispatch over the expert-parallel group,
grouped expert MLP, combine.

Numerics follow the reference: fp32 router (megatron/core/transformer/moe/router.py:25-471),
softmax -> top-k (or top-k -> softmax with ``moe_router_pre_softmax`` off), load-balancing loss
``sum_e(P_e * T_e) * E * coeff / (N^2 * k)`` (moe_utils.py:33-78), z-loss
``mean(logsumexp(logits)^2) * coeff`` (:134-146), auxiliary losses injected in backward by an
identity autograd function whose gradient is the current loss scale (:185-236), dropless by
default with optional capacity factor (:166,:529).  Dispatch is the all-to-all workflow of
token_dispatcher.py:332-788 (permute by expert, exchange by split sizes, sort by local expert,
expert compute, reverse); the all-gather dispatcher of :196 is kept for small EP sizes.

Expert weights are stored stacked - fc1 [E_local, 2f or f, h], fc2 [E_local, h, f] - and the
expert MLP runs on expert-sorted tokens through the ragged grouped product of
``ops/grouped_gemm.py``.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..config import TransformerConfig
from ..ops import core as ops
from ..ops import router as fused_router
from ..ops.grouped_gemm import grouped_linear
from ..parallel import state
from ..parallel.layers import _device, _init_sharded, set_tensor_model_parallel_attributes
from ..parallel.mappings import (all_to_all, gather_from_sequence_parallel_region,
                                 reduce_scatter_to_sequence_parallel_region)


# ----------------------------------------------------------------------------- aux loss plumbing
class MoEAuxLossAutoScaler(torch.autograd.Function):
    """Identity on ``output``; in backward, ``aux_loss`` receives gradient = current loss scale."""
    main_loss_backward_scale: Optional[torch.Tensor] = None

    @staticmethod
    def forward(ctx, output, aux_loss):
        ctx.save_for_backward(aux_loss)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (aux_loss,) = ctx.saved_tensors
        s = MoEAuxLossAutoScaler.main_loss_backward_scale
        if s is None:
            s = torch.ones(1, device=aux_loss.device)
        return grad_output, torch.ones_like(aux_loss) * s.to(aux_loss.device).reshape(()).to(aux_loss.dtype)

    @staticmethod
    def set_loss_scale(scale: torch.Tensor):
        MoEAuxLossAutoScaler.main_loss_backward_scale = scale


_MOE_METRICS = {}


def save_to_aux_losses_tracker(name: str, loss: torch.Tensor, layer_number: int, num_layers: int):
    t = _MOE_METRICS.setdefault(name, torch.zeros(num_layers, device=loss.device))
    t[layer_number - 1] += loss.detach()


def get_moe_metrics():
    return _MOE_METRICS


def clear_aux_losses_tracker():
    for t in _MOE_METRICS.values():
        t.zero_()


def track_moe_metrics(loss_scale: float, iteration: int, writer=None, total_loss_dict=None, per_layer=False):
    """Average tracked per-layer aux losses, reduce over PP/DP, log (reference: moe_utils.py:711)."""
    out = {}
    for name, t in _MOE_METRICS.items():
        v = t.clone() * loss_scale
        if dist.is_initialized() and state.model_parallel_is_initialized():
            if state.get_pipeline_model_parallel_world_size() > 1:
                dist.all_reduce(v, group=state.get_pipeline_model_parallel_group())
            if state.get_data_parallel_world_size() > 1:
                dist.all_reduce(v, group=state.get_data_parallel_group(), op=dist.ReduceOp.AVG)
        nz = (v != 0).sum().clamp(min=1)
        out[name] = (v.sum() / nz).item()
        if writer is not None:
            writer.add_scalar(name, out[name], iteration)
            if per_layer:
                for i, x in enumerate(v.tolist()):
                    writer.add_scalar(f"moe/{name}_layer_{i}", x, iteration)
        if total_loss_dict is not None:
            total_loss_dict[name] = total_loss_dict.get(name, 0.0) + out[name]
    clear_aux_losses_tracker()
    return out


# ----------------------------------------------------------------------------- routing math
def switch_load_balancing_loss_func(probs, tokens_per_expert, topk: int, coeff: float, num_tokens: int,
                                    num_experts: int):
    """sum_e(P_e * T_e) * E * coeff / (N^2 * k), P_e = summed probs, T_e = token counts."""
    agg = probs.sum(dim=0)
    return torch.sum(agg * tokens_per_expert) * (num_experts * coeff / (num_tokens * num_tokens * topk))


def z_loss_func(logits, coeff: float):
    return torch.mean(torch.square(torch.logsumexp(logits, dim=-1))) * coeff


def sinkhorn(cost, tol: float = 1e-4):
    cost = torch.exp(cost)
    d0 = torch.ones(cost.size(0), device=cost.device, dtype=cost.dtype)
    d1 = torch.ones(cost.size(1), device=cost.device, dtype=cost.dtype)
    eps, error, d1_old = 1e-8, 1e9, d1
    while error > tol:
        d0 = (1 / d0.size(0)) / (torch.sum(d1 * cost, 1) + eps)
        d1 = (1 / d1.size(0)) / (torch.sum(d0.unsqueeze(1) * cost, 0) + eps)
        error = torch.mean(torch.abs(d1_old - d1))
        d1_old = d1
    return d1 * cost * d0.unsqueeze(1)


def get_capacity(num_tokens: int, num_experts: int, capacity_factor: float, min_capacity: Optional[int] = None):
    cap = math.ceil(num_tokens / num_experts * capacity_factor)
    if min_capacity is not None and cap < min_capacity:
        cap = min_capacity
    return cap


def group_limited_topk(scores, topk, num_tokens, num_experts, num_groups, group_topk):
    """Device-limited routing: pick ``group_topk`` groups by the sum of their top
    ``topk // group_topk`` scores, then top-k inside them (reference: moe_utils.py:436)."""
    gs = scores.view(num_tokens, num_groups, -1).topk(topk // group_topk, dim=-1)[0].sum(dim=-1)
    gidx = torch.topk(gs, k=group_topk, dim=-1, sorted=False)[1]
    gmask = torch.zeros_like(gs).scatter_(1, gidx, 1)
    mask = gmask.unsqueeze(-1).expand(num_tokens, num_groups, num_experts // num_groups).reshape(num_tokens, -1)
    return torch.topk(scores.masked_fill(~mask.bool(), float("-inf")), k=topk, dim=-1)


def topk_softmax_with_capacity(logits, topk: int, capacity_factor=None, pad_to_capacity=False,
                               drop_policy="probs", use_pre_softmax=False, num_groups=None, group_topk=None,
                               scaling_factor=None, score_function="softmax", expert_bias=None):
    """Returns (probs [T, E] with zeros off the chosen experts, routing map [T, E] bool,
    tokens_per_expert [E]) (reference: moe_utils.py:529)."""
    T, E = logits.shape

    def pick(scores):
        if group_topk:
            return group_limited_topk(scores, topk, T, E, num_groups, group_topk)
        return torch.topk(scores, k=topk, dim=1)

    if score_function == "softmax":
        if use_pre_softmax:
            scores = torch.softmax(logits, dim=-1, dtype=torch.float32).type_as(logits)
            probs, idx = pick(scores)
        else:
            sc, idx = pick(logits)
            probs = torch.softmax(sc, dim=-1, dtype=torch.float32).type_as(logits)
    elif score_function == "sigmoid":
        scores = torch.sigmoid(logits.float()).type_as(logits)
        if expert_bias is not None:
            _, idx = pick(scores + expert_bias)
            probs = torch.gather(scores, dim=1, index=idx)
        else:
            probs, idx = pick(scores)
        probs = probs / (probs.sum(dim=-1, keepdim=True) + 1e-20) if topk > 1 else probs
    else:
        raise ValueError(f"unknown score function {score_function}")
    if scaling_factor:
        probs = probs * scaling_factor
    full = torch.zeros_like(logits).scatter(1, idx, probs)
    rmap = torch.zeros_like(logits).int().scatter(1, idx, 1).bool()
    tokens_per_expert = rmap.sum(dim=0)
    if capacity_factor is None:
        return full, rmap, tokens_per_expert
    cap = get_capacity(T * topk, E, capacity_factor)
    if drop_policy == "probs":
        _, cidx = torch.topk(full, k=min(cap, T), dim=0, sorted=False)
        cmask = torch.zeros_like(logits).scatter(0, cidx, 1).bool()
    elif drop_policy == "position":
        _, cidx = torch.topk(rmap.int(), k=min(cap, T), dim=0, sorted=False)
        cmask = torch.zeros_like(logits).scatter(0, cidx, 1).bool()
    else:
        raise ValueError(f"unknown drop policy {drop_policy}")
    if pad_to_capacity:
        final = cmask
    else:
        final = rmap & cmask
    return full * final, final, tokens_per_expert


def pad_routing_map(routing_map: torch.Tensor, pad_multiple: int) -> torch.Tensor:
    """Raise every expert's token count to the next multiple of ``pad_multiple`` by routing extra tokens (the first
    ones not yet routed to that expert) to it - FP8 grouped GEMMs want aligned row counts per expert.  The added
    entries carry probability zero, so the layer's output does not change
    (reference: megatron/core/transformer/moe/moe_utils.py:494 ``pad_routing_map``)."""
    rm = routing_map.bool()
    counts = rm.sum(dim=0)
    target = (counts + pad_multiple - 1) // pad_multiple * pad_multiple
    need = (target - counts).clamp(max=rm.shape[0] - counts)            # cannot exceed the tokens that exist
    # rank of every not-yet-routed token within its expert column: the first `need` of them are switched on
    free_rank = torch.cumsum((~rm).long(), dim=0)
    return rm | ((~rm) & (free_rank <= need.unsqueeze(0)))


class _RandomSTE(torch.autograd.Function):
    """Forward: uniform random scores of the same shape (the same on every rank that holds the same tokens is not
    required - each rank routes its own tokens); backward: identity."""

    @staticmethod
    def forward(ctx, logits):
        return torch.rand_like(logits)

    @staticmethod
    def backward(ctx, g):
        return g


class TopKRouter(nn.Module):
    def __init__(self, config: TransformerConfig, layer_number: int):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        self.num_experts, self.topk = config.num_moe_experts, config.moe_router_topk
        self.routing_type = config.moe_router_load_balancing_type
        self.weight = nn.Parameter(torch.empty(self.num_experts, config.hidden_size, device=_device(config),
                                               dtype=torch.float32))
        if config.perform_initialization:
            config.init_method(self.weight)
        self.weight.data = self.weight.data.to(config.params_dtype)
        self.weight.sequence_parallel = config.sequence_parallel
        if config.moe_router_enable_expert_bias:
            self.register_buffer("local_tokens_per_expert", torch.zeros(self.num_experts, device=_device(config)),
                                 persistent=False)
            self.register_buffer("expert_bias", torch.zeros(self.num_experts, device=_device(config)))
        else:
            self.expert_bias = None

    def gating(self, x):
        dt = {"fp32": torch.float32, "fp64": torch.float64}.get(self.config.moe_router_dtype, torch.float32)
        return F.linear(x.to(dt), self.weight.to(dt))

    def _aux(self, probs_for_loss, tokens_per_expert, activation, T):
        cfg = self.config
        group = state.get_tensor_and_context_parallel_group() if (
            state.model_parallel_is_initialized() and dist.is_initialized()
            and state.get_group_size("tp_cp") > 1) else None
        n_sub = state.get_group_size("tp_cp") if group is not None else 1
        tpe = tokens_per_expert.float()
        if group is not None:
            tpe = tpe.clone()
            dist.all_reduce(tpe, group=group)
        loss = switch_load_balancing_loss_func(probs_for_loss, tpe, self.topk, cfg.moe_aux_loss_coeff, T * n_sub,
                                               self.num_experts)
        if n_sub > 1:
            loss = loss * n_sub     # P_e is a local sum; the global product needs the group factor
        save_to_aux_losses_tracker("load_balancing_loss", loss / max(cfg.moe_aux_loss_coeff, 1e-30),
                                   self.layer_number, cfg.num_layers)
        return MoEAuxLossAutoScaler.apply(activation, loss)

    def _fused_eligible(self, logits) -> bool:
        """One CUDA pass for scores, top-k, map and loss statistics (``ops/router.py``): GPU tensors, no capacity
        dropping, no group-limited choice, plain or aux-loss balancing.  ``MLB_FUSED_ROUTER=0`` turns it off."""
        cfg = self.config
        return (logits.is_cuda and os.environ.get("MLB_FUSED_ROUTER", "1") != "0"
                and self.routing_type in ("aux_loss", "none") and cfg.moe_expert_capacity_factor is None
                and not cfg.moe_router_group_topk and logits.dtype == torch.float32
                and self.num_experts <= fused_router.MAX_EXPERTS
                and cfg.moe_router_score_function in ("softmax", "sigmoid")
                and not (cfg.moe_router_padding_for_fp8 and cfg.fp8))

    def _forward_fused(self, logits):
        cfg = self.config
        train = self.training
        aux_c = cfg.moe_aux_loss_coeff if (train and self.routing_type == "aux_loss") else 0.0
        z_c = cfg.moe_z_loss_coeff if (train and cfg.moe_z_loss_coeff is not None) else 0.0
        group = None
        if aux_c and state.model_parallel_is_initialized() and dist.is_initialized() \
                and state.get_group_size("tp_cp") > 1:
            group = state.get_tensor_and_context_parallel_group()
        probs, rmap, _tpe, aux, z = fused_router.fused_topk_router(
            logits, self.topk, fused_router.router_mode(cfg.moe_router_score_function, cfg.moe_router_pre_softmax),
            cfg.moe_router_topk_scaling_factor, self.expert_bias, aux_c, z_c, group,
            lambda: MoEAuxLossAutoScaler.main_loss_backward_scale)
        if aux_c:
            save_to_aux_losses_tracker("load_balancing_loss", aux / aux_c, self.layer_number, cfg.num_layers)
        if z_c:
            save_to_aux_losses_tracker("z_loss", z / z_c, self.layer_number, cfg.num_layers)
        if self.expert_bias is not None and train:
            with torch.no_grad():
                self.local_tokens_per_expert += _tpe
        return probs, rmap

    def forward(self, hidden):
        cfg = self.config
        h = hidden.reshape(-1, hidden.shape[-1])
        if self.training and cfg.moe_input_jitter_eps is not None:
            eps = cfg.moe_input_jitter_eps
            h = h * torch.empty_like(h).uniform_(1.0 - eps, 1.0 + eps)
        logits = self.gating(h)
        if cfg.moe_router_force_load_balancing:
            # benchmarking aid: routing by random scores spreads the tokens evenly over the experts whatever the
            # router has learnt; gradients pass straight through (reference: moe_utils.py RandomSTE)
            logits = _RandomSTE.apply(logits)
        T = logits.shape[0]
        if self._fused_eligible(logits):
            return self._forward_fused(logits)
        if cfg.moe_z_loss_coeff is not None and self.training:
            z = z_loss_func(logits, cfg.moe_z_loss_coeff)
            logits = MoEAuxLossAutoScaler.apply(logits, z)
            save_to_aux_losses_tracker("z_loss", z / cfg.moe_z_loss_coeff, self.layer_number, cfg.num_layers)
        if self.routing_type == "sinkhorn":
            if self.training:
                with torch.no_grad():
                    norm = sinkhorn(logits.float())
                    _, idx = torch.topk(norm, k=self.topk, dim=1)
                act = torch.sigmoid(logits) if self.topk == 1 else torch.softmax(logits, -1, dtype=torch.float32)
                sc = torch.gather(act, 1, idx)
            else:
                act = torch.sigmoid(logits) if self.topk == 1 else torch.softmax(logits, -1, dtype=torch.float32)
                sc, idx = torch.topk(act, k=self.topk, dim=1)
            probs = torch.zeros_like(logits).scatter(1, idx, sc.type_as(logits))
            rmap = torch.zeros_like(logits).int().scatter(1, idx, 1).bool()
            return probs, rmap
        probs, rmap, tpe = topk_softmax_with_capacity(
            logits, self.topk, cfg.moe_expert_capacity_factor, cfg.moe_pad_expert_input_to_capacity,
            cfg.moe_token_drop_policy, cfg.moe_router_pre_softmax, cfg.moe_router_num_groups,
            cfg.moe_router_group_topk, cfg.moe_router_topk_scaling_factor, cfg.moe_router_score_function,
            self.expert_bias)
        if cfg.moe_router_padding_for_fp8 and cfg.fp8:
            rmap = pad_routing_map(rmap, 16)          # probabilities of the added entries stay zero
        if self.training and cfg.moe_aux_loss_coeff > 0 and self.routing_type in ("aux_loss", "seq_aux_loss"):
            scores = torch.softmax(logits, dim=-1, dtype=torch.float32) if cfg.moe_router_score_function == "softmax" \
                else torch.sigmoid(logits.float())
            probs = self._aux(scores, tpe, probs, T)
        if self.expert_bias is not None and self.training:
            with torch.no_grad():
                self.local_tokens_per_expert += rmap.sum(dim=0)
        return probs, rmap


def get_updated_expert_bias(tokens_per_expert, expert_bias, rate):
    """Aux-loss-free balancing: raise the bias of under-loaded experts (reference: moe_utils.py:787)."""
    with torch.no_grad():
        if dist.is_initialized() and state.model_parallel_is_initialized():
            dist.all_reduce(tokens_per_expert, group=state.get_tensor_and_data_parallel_group(True))
        avg = tokens_per_expert.sum(dim=-1, keepdim=True) / tokens_per_expert.shape[-1]
        return expert_bias + torch.sign(avg - tokens_per_expert) * rate


# ----------------------------------------------------------------------------- permutation
def permute(tokens, routing_map):
    """[T, h], [T, E] bool -> expert-major token copies [sum(map), h] and the source row of each."""
    T, E = routing_map.shape
    rm = routing_map.t().contiguous()                          # [E, T]
    token_idx = torch.arange(T, device=tokens.device).unsqueeze(0).expand(E, -1)
    sorted_indices = token_idx.masked_select(rm)
    return tokens.index_select(0, sorted_indices), sorted_indices


def unpermute(permuted, sorted_indices, shape, probs=None, routing_map=None):
    """Inverse of :func:`permute` with optional per-copy prob weighting, summing copies per token."""
    T, h = shape
    if probs is not None:
        w = probs.t().contiguous().masked_select(routing_map.t().contiguous())
        permuted = permuted * w.unsqueeze(-1).to(permuted.dtype)
    out = torch.zeros(T, h, dtype=permuted.dtype, device=permuted.device)
    out.index_add_(0, sorted_indices, permuted)
    return out


def sort_chunks_by_idxs(x, split_sizes: List[int], idxs: List[int]):
    chunks = torch.split(x, split_sizes, dim=0)
    return torch.cat([chunks[i] for i in idxs], dim=0)


# ----------------------------------------------------------------------------- experts
class GroupedMLP(nn.Module):
    """E_local experts evaluated on expert-sorted tokens with ragged grouped GEMMs."""

    def __init__(self, num_local_experts: int, config: TransformerConfig):
        super().__init__()
        self.config, self.E = config, num_local_experts
        init = state.model_parallel_is_initialized()
        etp = state.get_expert_tensor_parallel_world_size() if init else 1
        etp_rank = state.get_expert_tensor_parallel_rank() if init else 0
        ep_rank = state.get_expert_model_parallel_rank() if init else 0
        f = config.moe_ffn_hidden_size
        self.gated = config.gated_linear_unit
        fc1_out = f * (2 if self.gated else 1)
        dev = _device(config)
        self.f_local = f // etp
        self.weight1 = nn.Parameter(torch.empty(self.E, fc1_out // etp, config.hidden_size, device=dev,
                                                dtype=config.params_dtype))
        self.weight2 = nn.Parameter(torch.empty(self.E, config.hidden_size, f // etp, device=dev,
                                                dtype=config.params_dtype))
        for e in range(self.E):
            _init_sharded(self.weight1[e], (fc1_out, config.hidden_size), 0, config.init_method, config, etp_rank, etp,
                          2 if self.gated else 1, is_expert=True)
            _init_sharded(self.weight2[e], (config.hidden_size, f), 1, config.output_layer_init_method, config,
                          etp_rank, etp, 1, is_expert=True)
        for w, dim in ((self.weight1, 1), (self.weight2, 2)):
            set_tensor_model_parallel_attributes(w, True, dim, 1)
            w.allreduce = not (config.expert_model_parallel_size > 1)
        self.etp = etp
        self.num_global_offset = ep_rank * self.E

    def forward(self, tokens, tokens_per_expert, probs=None):
        """tokens [N, h] sorted by local expert; tokens_per_expert [E_local] (host list or tensor)."""
        h1 = grouped_linear(tokens, self.weight1, tokens_per_expert)
        if self.gated:
            a = ops.swiglu(h1) if self.config.activation_func in ("silu", "swiglu") else \
                (F.gelu(h1.chunk(2, -1)[0]) * h1.chunk(2, -1)[1])
        else:
            a = ops.bias_gelu(h1, None) if self.config.activation_func == "gelu" else F.relu(h1)
        if probs is not None:
            a = a * probs.unsqueeze(-1).to(a.dtype)
        return grouped_linear(a, self.weight2, tokens_per_expert), None


class SequentialMLP(nn.Module):
    """One ordinary MLP module per local expert, applied to that expert's slice of the sorted tokens
    (reference: experts.py:988; parameter names ``local_experts.<e>.linear_fc{1,2}``).  Used when
    ``moe_grouped_gemm`` is off, e.g. for checkpoints converted expert by expert."""

    def __init__(self, num_local_experts: int, config: TransformerConfig):
        super().__init__()
        from .transformer import MLP
        self.E = num_local_experts
        self.local_experts = nn.ModuleList([MLP(config, ffn_hidden_size=config.moe_ffn_hidden_size, is_expert=True)
                                            for _ in range(num_local_experts)])

    def forward(self, tokens, tokens_per_expert):
        splits = [int(v) for v in (tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else tokens_per_expert)]
        outs, o = [], 0
        for e, n in enumerate(splits):
            x = tokens[o:o + n]
            y, b = self.local_experts[e](x)
            outs.append(y if b is None else y + b)
            o += n
        return (torch.cat(outs, dim=0) if outs else tokens.new_zeros(0, tokens.shape[-1])), None


class SharedExpertMLP(nn.Module):
    """Dense MLP applied to every token next to the routed experts (reference: shared_experts.py:26)."""

    def __init__(self, config: TransformerConfig):
        super().__init__()
        from .transformer import MLP
        self.mlp = MLP(config, ffn_hidden_size=config.moe_shared_expert_intermediate_size)

    def forward(self, x):
        out, bias = self.mlp(x)
        return out if bias is None else out + bias


# ----------------------------------------------------------------------------- dispatchers
class MoEAlltoAllTokenDispatcher:
    """permute -> all-to-all(EP) -> sort by local expert -> experts -> reverse."""

    def __init__(self, num_local_experts: int, config: TransformerConfig):
        self.config, self.E_local = config, num_local_experts
        init = state.model_parallel_is_initialized() and dist.is_initialized()
        self.ep_group = state.get_expert_model_parallel_group() if init else None
        self.ep = state.get_expert_model_parallel_world_size() if init else 1
        self.E = config.num_moe_experts

    def dispatch(self, hidden, probs, routing_map):
        self.shape = hidden.shape
        h = hidden.reshape(-1, hidden.shape[-1])
        self.T = h.shape[0]
        self.routing_map, self.probs = routing_map, probs
        permuted, self.sorted_indices = permute(h, routing_map)
        local_counts = routing_map.sum(dim=0).to(torch.int64)              # [E]
        if self.ep > 1:
            flat_counts = torch.empty(self.ep * self.E, dtype=torch.int64, device=h.device)
            dist.all_gather_into_tensor(flat_counts, local_counts.contiguous(), group=self.ep_group)
            all_counts = flat_counts.view(self.ep, self.E)
            r = dist.get_rank(self.ep_group)
            mine = all_counts[:, r * self.E_local:(r + 1) * self.E_local]    # [ep, E_local]: from each source rank
            # one host read per layer: split sizes are needed by the collective
            sizes = torch.cat((local_counts.view(self.ep, self.E_local).sum(1), mine.sum(1), mine.reshape(-1))).tolist()
            self.input_splits = [int(x) for x in sizes[:self.ep]]
            self.output_splits = [int(x) for x in sizes[self.ep:2 * self.ep]]
            per_src = [int(x) for x in sizes[2 * self.ep:]]
            recv = all_to_all(self.ep_group, permuted, self.output_splits, self.input_splits)
            # received layout: [src rank][local expert]; regroup to [local expert][src rank]
            if self.E_local > 1:
                order = [s * self.E_local + e for e in range(self.E_local) for s in range(self.ep)]
                recv = sort_chunks_by_idxs(recv, per_src, order)
                self._restore = (
                    [per_src[i] for i in order],
                    [order.index(i) for i in range(len(order))])
            else:
                self._restore = None
            tpe = mine.sum(0)
        else:
            recv, tpe, self._restore = permuted, local_counts, None
        return recv, tpe

    def combine(self, expert_out):
        x = expert_out
        if self._restore is not None:
            x = sort_chunks_by_idxs(x, self._restore[0], self._restore[1])
        if self.ep > 1:
            x = all_to_all(self.ep_group, x, self.input_splits, self.output_splits)
        out = unpermute(x, self.sorted_indices, (self.T, self.shape[-1]), self.probs, self.routing_map)
        return out.view(self.shape)


_FUSED_COMM = {}


class MoEFusedPeerDispatcher(MoEAlltoAllTokenDispatcher):
    """Dispatch / combine as single kernels over NVLink peer memory (``ops/moe_fused.py``): permute + all-to-all
    and all-to-all + un-permute + prob weighting, each one launch.  Used for CUDA tensors with expert
    parallelism and a dropless router; otherwise behaves like the all-to-all dispatcher."""

    def _comm(self, T, hdim, dtype):
        from ..ops.moe_fused import FusedMoEComm
        key = (id(self.ep_group), T, hdim, dtype, self.config.moe_router_topk)
        if key not in _FUSED_COMM:
            _FUSED_COMM[key] = FusedMoEComm(self.ep_group, T, self.config.moe_router_topk, hdim, self.E, dtype)
        return _FUSED_COMM[key]

    def _use_fused(self, h):
        return h.is_cuda and self.ep > 1 and self.config.moe_expert_capacity_factor is None and \
            h.dtype in (torch.bfloat16, torch.float16)

    def dispatch(self, hidden, probs, routing_map):
        h = hidden.reshape(-1, hidden.shape[-1])
        self.fused = self._use_fused(h)
        if not self.fused:
            return super().dispatch(hidden, probs, routing_map)
        from ..ops.moe_fused import fused_dispatch
        self.shape, self.T = hidden.shape, h.shape[0]
        rm = routing_map.t().contiguous()
        # dropless top-k routing: exactly T * topk copies, so the (expert, token) pairs can be listed without the
        # host learning a data-dependent size (row-major order of the [E, T] map = expert-major copy order)
        pairs = rm.nonzero_static(size=self.T * self.config.moe_router_topk)
        sorted_indices = pairs[:, 1].contiguous()
        self.comm = self._comm(self.T, h.shape[1], h.dtype)
        self.plan = self.comm.plan(routing_map, sorted_indices)
        self.copy_probs = probs.t()[pairs[:, 0], pairs[:, 1]]
        recv = fused_dispatch(h, self.comm, self.plan)
        return recv, self.plan["tokens_per_local_expert"]

    def combine(self, expert_out):
        if not self.fused:
            return super().combine(expert_out)
        from ..ops.moe_fused import fused_combine
        out = fused_combine(expert_out, self.copy_probs, self.comm, self.plan, self.T)
        return out.view(self.shape)


class MoEAllGatherTokenDispatcher:
    """Gather every rank's tokens, run the local experts on the ones routed here, reduce-scatter
    the outputs back (reference: token_dispatcher.py:196)."""

    def __init__(self, num_local_experts: int, config: TransformerConfig):
        self.config, self.E_local = config, num_local_experts
        init = state.model_parallel_is_initialized() and dist.is_initialized()
        self.group = state.get_expert_model_parallel_group() if init else None
        self.ep = state.get_expert_model_parallel_world_size() if init else 1

    def dispatch(self, hidden, probs, routing_map):
        self.shape = hidden.shape
        h = hidden.reshape(-1, hidden.shape[-1])
        if self.ep > 1:
            h = gather_from_sequence_parallel_region(h, True, self.group)
            probs = gather_from_sequence_parallel_region(probs, True, self.group)
            routing_map = gather_from_sequence_parallel_region(routing_map.to(torch.uint8), False, self.group).bool()
        r = dist.get_rank(self.group) if self.ep > 1 else 0
        sl = slice(r * self.E_local, (r + 1) * self.E_local)
        self.local_map = routing_map[:, sl].contiguous()
        self.local_probs = probs[:, sl].contiguous()
        self.T = h.shape[0]
        permuted, self.sorted_indices = permute(h, self.local_map)
        return permuted, self.local_map.sum(dim=0).to(torch.int64)

    def combine(self, expert_out):
        out = unpermute(expert_out, self.sorted_indices, (self.T, self.shape[-1]), self.local_probs, self.local_map)
        if self.ep > 1:
            out = reduce_scatter_to_sequence_parallel_region(out, self.group)
        return out.view(self.shape)


# ----------------------------------------------------------------------------- layer
class MoELayer(nn.Module):
    def __init__(self, config: TransformerConfig, layer_number: int):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        ep = state.get_expert_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.E_local = config.num_moe_experts // ep
        self.router = TopKRouter(config, layer_number)
        self.experts = GroupedMLP(self.E_local, config) if config.moe_grouped_gemm else SequentialMLP(self.E_local, config)
        kind = config.moe_token_dispatcher_type
        if kind == "flex":
            self.token_dispatcher = MoEFusedPeerDispatcher(self.E_local, config)
        elif kind in ("alltoall", "alltoall_seq"):
            self.token_dispatcher = MoEAlltoAllTokenDispatcher(self.E_local, config)
        elif kind == "allgather":
            self.token_dispatcher = MoEAllGatherTokenDispatcher(self.E_local, config)
        else:
            raise ValueError(f"unknown token dispatcher {kind}")
        self.shared_experts = SharedExpertMLP(config) if config.moe_shared_expert_intermediate_size else None

    def forward(self, hidden):
        probs, rmap = self.router(hidden)
        if self.config.moe_apply_probs_on_input:
            # top-1 routing with the weight applied before the expert: E(p x) instead of p E(x)
            hidden = (hidden.reshape(-1, hidden.shape[-1]) * probs.sum(dim=-1, keepdim=True).to(hidden.dtype)).view_as(hidden)
            probs = rmap.to(probs.dtype)
        tokens, tpe = self.token_dispatcher.dispatch(hidden, probs, rmap)
        out, _ = self.experts(tokens, tpe)
        out = self.token_dispatcher.combine(out)
        if self.shared_experts is not None:
            out = out + self.shared_experts(hidden)
        return out, None
