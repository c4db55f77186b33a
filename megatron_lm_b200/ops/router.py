"""Fused mixture-of-experts routing: scores, top-k, dense probabilities / routing map and the statistics of the
load-balancing and z losses in one CUDA pass (``csrc/router.cu``), with one backward pass that combines the gradient
of the token weighting, of the load-balancing loss and of the z loss.

``fused_topk_router(logits, ...)`` returns ``(probs [T, E], routing_map [T, E] bool, tokens_per_expert [E],
aux_loss, z_loss)``; the two losses are detached values for logging - their gradients reach ``logits`` through
the backward of ``probs``, scaled by ``loss_scale`` (a tensor read at backward time, the pipeline schedule's
loss scale).  CPU tensors take the plain PyTorch body, which is also the numerical reference of the kernel.
Reference: megatron/core/transformer/moe/moe_utils.py:529 (routing), :35 (load-balancing loss), :107 (z loss),
:440 (MoEAuxLossAutoScaler).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib

_lib.register_signatures({
    "mlb_moe_router_fwd": "ppppppp" "iiii" "f" "p",
    "mlb_moe_router_bwd": "ppppp" "iiii" "ff" "p",
})

MODES = {"softmax_post": 0, "softmax_pre": 1, "sigmoid": 2}
MAX_EXPERTS = 1024


def router_mode(score_function: str, pre_softmax: bool) -> str:
    if score_function == "sigmoid":
        return "sigmoid"
    if score_function != "softmax":
        raise ValueError(f"unknown score function {score_function}")
    return "softmax_pre" if pre_softmax else "softmax_post"


def _reference(logits, topk, mode, scale, bias):
    """Dense probs / map / counts / score sums / sum of logsumexp^2 in plain PyTorch (fp32)."""
    lf = logits.float()
    if mode == "sigmoid":
        full = torch.sigmoid(lf)
        pick = full + bias.float() if bias is not None else full
        _, idx = torch.topk(pick, topk, dim=1)
        p = torch.gather(full, 1, idx)
        if topk > 1:
            p = p / (p.sum(dim=-1, keepdim=True) + 1e-20)
    else:
        full = torch.softmax(lf, dim=-1)
        if mode == "softmax_pre":
            p, idx = torch.topk(full, topk, dim=1)
        else:
            sc, idx = torch.topk(lf, topk, dim=1)
            p = torch.softmax(sc, dim=-1)
    probs = torch.zeros_like(lf).scatter(1, idx, p * scale)
    rmap = torch.zeros_like(lf, dtype=torch.bool).scatter(1, idx, True)
    zsum = torch.logsumexp(lf, dim=-1).square().sum()
    return probs, rmap, rmap.sum(dim=0).int(), full.sum(dim=0), zsum


def _scale_value(loss_scale, device) -> torch.Tensor:
    """``loss_scale`` is a tensor, a zero-argument callable returning one (read at backward time), or None."""
    v = loss_scale() if callable(loss_scale) else loss_scale
    if v is None:
        return torch.ones((), device=device, dtype=torch.float32)
    return v.to(device=device, dtype=torch.float32).reshape(())


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, topk, mode, scale, aux_const, z_coeff, stat_group, n_sub, loss_scale):
        lg = logits.float().contiguous()
        T, E = lg.shape
        probs = torch.empty_like(lg)
        rmap = torch.empty(T, E, dtype=torch.uint8, device=lg.device)
        stats = torch.zeros(2 * E + 1, dtype=torch.float32, device=lg.device)
        tpe = torch.zeros(E, dtype=torch.int32, device=lg.device)
        bf = None if bias is None else bias.float().contiguous()
        _lib.check(_lib.lib().mlb_moe_router_fwd(lg.data_ptr(), _lib.ptr(bf), probs.data_ptr(), rmap.data_ptr(),
                                                 tpe.data_ptr(), stats.data_ptr(), stats[2 * E:].data_ptr(), T, E,
                                                 topk, MODES[mode], float(scale), _lib.stream()), "moe_router_fwd")
        score_sum, zsum = stats[:E], stats[2 * E]
        tpe_f = tpe.float()
        if stat_group is not None:
            torch.distributed.all_reduce(tpe_f, group=stat_group)
        # loss = sum_e P_e T_e * aux_const, P_e local score sums, T_e counts over the statistics group
        aux = (score_sum * tpe_f).sum() * (aux_const * n_sub)
        z = zsum * (z_coeff / max(T, 1))
        ctx.save_for_backward(lg, rmap, tpe_f)
        ctx.cfg = (topk, mode, float(scale), float(aux_const) * n_sub, float(z_coeff), loss_scale, logits.dtype)
        ctx.mark_non_differentiable(rmap, tpe, aux, z)
        return probs, rmap, tpe, aux, z

    @staticmethod
    def backward(ctx, dprobs, _dm, _dt, _da, _dz):
        lg, rmap, tpe_f = ctx.saved_tensors
        topk, mode, scale, aux_const, z_coeff, loss_scale, in_dtype = ctx.cfg
        T, E = lg.shape
        ls = _scale_value(loss_scale, lg.device)
        coef = None
        if aux_const != 0.0:
            coef = (tpe_f * aux_const * ls).contiguous()
        zc = 0.0
        if z_coeff != 0.0:
            zc = float(z_coeff) * float(ls) / max(T, 1)
        dl = torch.empty_like(lg)
        dp = dprobs.float().contiguous()
        _lib.check(_lib.lib().mlb_moe_router_bwd(lg.data_ptr(), rmap.data_ptr(), dp.data_ptr(), _lib.ptr(coef),
                                                 dl.data_ptr(), T, E, topk, MODES[mode], scale, zc, _lib.stream()),
                   "moe_router_bwd")
        return dl.to(in_dtype), None, None, None, None, None, None, None, None, None


class _AuxGrad(torch.autograd.Function):
    """CPU body: attaches the loss gradients to ``probs`` the way the CUDA backward does internally."""

    @staticmethod
    def forward(ctx, probs, loss, loss_scale):
        ctx.save_for_backward(loss)
        ctx.loss_scale = loss_scale
        return probs

    @staticmethod
    def backward(ctx, g):
        (loss,) = ctx.saved_tensors
        return g, torch.ones_like(loss) * _scale_value(ctx.loss_scale, loss.device).to(loss.dtype), None


def fused_topk_router(logits: torch.Tensor, topk: int, mode: str = "softmax_post", scale: Optional[float] = None,
                      expert_bias: Optional[torch.Tensor] = None, aux_coeff: float = 0.0, z_coeff: float = 0.0,
                      stat_group=None, loss_scale=None):
    """See the module docstring.  ``aux_coeff`` / ``z_coeff`` of 0 leave that loss out; ``stat_group`` is the
    process group over which the token counts of the load-balancing loss are summed (the ranks that hold
    different tokens of the same sequences)."""
    T, E = logits.shape
    if E > MAX_EXPERTS:
        raise ValueError(f"fused router supports at most {MAX_EXPERTS} experts, got {E}")
    sc = 1.0 if not scale else float(scale)
    n_sub = torch.distributed.get_world_size(stat_group) if stat_group is not None else 1
    n_tok = T * n_sub
    aux_const = aux_coeff * E / (n_tok * n_tok * topk) if aux_coeff else 0.0
    if logits.is_cuda:
        probs, rmap, tpe, aux, z = _RouterFn.apply(logits, expert_bias, topk, mode, sc, aux_const, z_coeff or 0.0,
                                                   stat_group, n_sub, loss_scale)
        return probs, rmap.view(torch.bool), tpe, aux, z
    probs, rmap, tpe, score_sum, zsum = _reference(logits, topk, mode, sc, expert_bias)
    tpe_f = tpe.float()
    if stat_group is not None:
        torch.distributed.all_reduce(tpe_f, group=stat_group)
    aux = (score_sum * tpe_f).sum() * (aux_const * n_sub)
    z = zsum * ((z_coeff or 0.0) / max(T, 1))
    if aux_coeff:
        probs = _AuxGrad.apply(probs, aux, loss_scale)
    if z_coeff:
        probs = _AuxGrad.apply(probs, z, loss_scale)
    return probs.to(logits.dtype) if logits.dtype != torch.float32 else probs, rmap, tpe, aux.detach(), z.detach()
