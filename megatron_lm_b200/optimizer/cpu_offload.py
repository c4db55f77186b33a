"""Optimizer whose state (and update) for a fraction of the parameters lives in host memory.

Reference: megatron/core/optimizer/cpu_offloading/hybrid_optimizer.py (``HybridDeviceOptimizer`` :14;
split by ``offload_fraction`` :251, D2H gradients / H2D parameters :117, ``step`` :150).

Parameters are assigned to the host side in order until ``offload_fraction`` of all elements is
covered.  For those, fp32 master weights and Adam moments are pinned host tensors; each step copies
their gradients device->host on a side stream (overlapping the device-side update of the rest),
runs the host AdamW, and copies the updated weights back host->device, again asynchronously.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch


def _pin(t: torch.Tensor) -> torch.Tensor:
    if torch.cuda.is_available():
        try:
            return t.pin_memory()
        except RuntimeError:
            return t
    return t


class HybridDeviceOptimizer(torch.optim.Optimizer):
    def __init__(self, params, offload_fraction: float = 0.5, cpu_optimizer_cls=None, gpu_optimizer_cls=None,
                 param_update_in_fp32: bool = True, pin_cpu_grads: bool = True, pin_cpu_params: bool = True,
                 overlap_cpu_optimizer_d2h_h2d: bool = True, **kwargs):
        groups = list(params)
        if groups and not isinstance(groups[0], dict):
            groups = [{"params": groups}]
        defaults = dict(kwargs)
        super().__init__(groups, defaults)
        self.offload_fraction = offload_fraction
        self.overlap = overlap_cpu_optimizer_d2h_h2d
        cpu_cls = cpu_optimizer_cls or torch.optim.AdamW
        gpu_cls = gpu_optimizer_cls or torch.optim.AdamW
        total = sum(p.numel() for g in self.param_groups for p in g["params"])
        budget = int(total * offload_fraction)
        self.cpu_copy: Dict[torch.nn.Parameter, torch.Tensor] = {}
        self.gpu_master: Dict[torch.nn.Parameter, torch.Tensor] = {}
        cpu_groups, gpu_groups = [], []
        used = 0
        for gi, g in enumerate(self.param_groups):
            opts = {k: v for k, v in g.items() if k != "params"}
            opts["outer_group"] = gi                      # which of this optimizer's groups an inner group mirrors
            cg, gg = dict(opts, params=[]), dict(opts, params=[])
            for p in g["params"]:
                if used + p.numel() <= budget:
                    used += p.numel()
                    host = _pin(p.detach().float().cpu().clone()) if pin_cpu_params else p.detach().float().cpu().clone()
                    host.grad = _pin(torch.zeros_like(host)) if pin_cpu_grads else torch.zeros_like(host)
                    self.cpu_copy[p] = host
                    cg["params"].append(host)
                else:
                    if param_update_in_fp32 and p.dtype != torch.float32:
                        m = p.detach().float().clone()
                        m.grad = torch.zeros_like(m)
                        self.gpu_master[p] = m
                        gg["params"].append(m)
                    else:
                        gg["params"].append(p)
            if cg["params"]:
                cpu_groups.append(cg)
            if gg["params"]:
                gpu_groups.append(gg)
        self.cpu_optimizer = cpu_cls(cpu_groups, **kwargs) if cpu_groups else None
        self.gpu_optimizer = gpu_cls(gpu_groups, **kwargs) if gpu_groups else None
        self._stream = torch.cuda.Stream() if (torch.cuda.is_available() and self.overlap) else None

    @property
    def sub_optimizers(self):
        return [o for o in (self.cpu_optimizer, self.gpu_optimizer) if o is not None]

    def _sync_hyper(self):
        """lr / weight decay set on this optimizer's groups by a scheduler reach the inner optimizers."""
        for inner in self.sub_optimizers:
            for ig in inner.param_groups:
                g = self.param_groups[ig.get("outer_group", 0)]
                for k in ("lr", "weight_decay", "betas", "eps"):
                    if k in g:
                        ig[k] = g[k]

    def _grad_of(self, p):
        g = getattr(p, "main_grad", None)
        return g if g is not None else p.grad

    @torch.no_grad()
    def step(self, closure=None):
        self._sync_hyper()
        cur = torch.cuda.current_stream() if self._stream is not None else None
        # 1. gradients of the offloaded part leave for the host
        if self._stream is not None:
            self._stream.wait_stream(cur)
        ctx = torch.cuda.stream(self._stream) if self._stream is not None else _null()
        with ctx:
            for p, host in self.cpu_copy.items():
                g = self._grad_of(p)
                if g is not None:
                    host.grad.copy_(g.detach().float().reshape(host.shape), non_blocking=True)
        # 2. the device-resident part updates meanwhile
        if self.gpu_optimizer is not None:
            for p, m in self.gpu_master.items():
                g = self._grad_of(p)
                if g is not None:
                    m.grad.copy_(g.detach().float().reshape(m.shape))
            # parameters the device optimizer updates in place take their gradient from main_grad when the
            # model keeps gradients in the data-parallel buffers (``.grad`` is then empty)
            masters = {id(m) for m in self.gpu_master.values()}
            direct = [p for g in self.gpu_optimizer.param_groups for p in g["params"] if id(p) not in masters]
            for p in direct:
                mg = getattr(p, "main_grad", None)
                if mg is not None:
                    p.grad = mg.to(p.dtype).reshape(p.shape)
            self.gpu_optimizer.step()
            for p in direct:
                if getattr(p, "main_grad", None) is not None:
                    p.grad = None
            for p, m in self.gpu_master.items():
                p.data.copy_(m.to(p.dtype))
        # 3. host update, then weights return
        if self._stream is not None:
            self._stream.synchronize()
        if self.cpu_optimizer is not None:
            self.cpu_optimizer.step()
            with ctx:
                for p, host in self.cpu_copy.items():
                    p.data.copy_(host.to(p.dtype).reshape(p.shape), non_blocking=True)
            if self._stream is not None:
                cur.wait_stream(self._stream)
        return None

    def zero_grad(self, set_to_none: bool = True):
        for g in self.param_groups:
            for p in g["params"]:
                p.grad = None

    def state_dict(self):
        return {"cpu": None if self.cpu_optimizer is None else self.cpu_optimizer.state_dict(),
                "gpu": None if self.gpu_optimizer is None else self.gpu_optimizer.state_dict(),
                "cpu_master": [h.clone() for h in self.cpu_copy.values()],
                "gpu_master": [m.clone() for m in self.gpu_master.values()]}

    def load_state_dict(self, sd):
        if self.cpu_optimizer is not None and sd["cpu"] is not None:
            self.cpu_optimizer.load_state_dict(sd["cpu"])
        if self.gpu_optimizer is not None and sd["gpu"] is not None:
            self.gpu_optimizer.load_state_dict(sd["gpu"])
        for h, s in zip(self.cpu_copy.values(), sd["cpu_master"]):
            h.copy_(s)
        for m, s in zip(self.gpu_master.values(), sd["gpu_master"]):
            m.copy_(s)


class _null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


class OffloadedOptimizer:
    """``HybridDeviceOptimizer`` behind the training loop's optimizer surface, for models wrapped in the replicated
    data-parallel buffers: gradients are read from ``main_grad`` after the data-parallel reduction, the global norm
    (over the model-parallel group) clips them, weight-decay groups follow the usual bias / 1-d rule.
    Selected by ``--optimizer-cpu-offload`` with ``--optimizer-offload-fraction`` (reference:
    megatron/core/optimizer/__init__.py:330-370 building HybridDeviceOptimizer)."""

    def __init__(self, model_chunks, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 clip_grad: float = 0.0, offload_fraction: float = 1.0, model_parallel_group=None):
        named = [(n, p) for m in model_chunks for n, p in m.named_parameters() if p.requires_grad]
        decay = [p for n, p in named if not (n.endswith(".bias") or p.dim() == 1)]
        no_decay = [p for n, p in named if (n.endswith(".bias") or p.dim() == 1)]
        groups = [g for g in (dict(params=decay, weight_decay=weight_decay, wd_mult=1.0),
                              dict(params=no_decay, weight_decay=0.0, wd_mult=0.0)) if g["params"]]
        self.opt = HybridDeviceOptimizer(groups, offload_fraction=offload_fraction, lr=lr, betas=betas, eps=eps,
                                         weight_decay=weight_decay)
        for g in self.opt.param_groups:
            g.setdefault("max_lr", lr)
            g.setdefault("min_lr", 0.0)
        self.params = [p for _, p in named]
        self.clip, self.mp_group = clip_grad, model_parallel_group

    @property
    def param_groups(self):
        return self.opt.param_groups

    def zero_grad(self, set_to_none: bool = True):
        self.opt.zero_grad(set_to_none)

    def scale_loss(self, loss):
        return loss

    def get_loss_scale(self) -> torch.Tensor:
        return torch.ones(1, dtype=torch.float32)

    @torch.no_grad()
    def step(self):
        import torch.distributed as dist
        from ..parallel import state
        for g in self.opt.param_groups:                       # the scheduler writes one decay for all groups
            g["weight_decay"] = g["weight_decay"] * g.get("wd_mult", 1.0)
        tp0 = (not state.model_parallel_is_initialized()) or state.get_tensor_model_parallel_rank() == 0
        dev = self.params[0].device
        tot = torch.zeros(1, dtype=torch.float32, device=dev)
        grads = []
        for p in self.params:
            g = getattr(p, "main_grad", None)
            g = g if g is not None else p.grad
            if g is None:
                continue
            grads.append(g)
            if getattr(p, "tensor_model_parallel", False) or tp0:
                tot += g.float().pow(2).sum()
        if self.mp_group is not None:
            dist.all_reduce(tot, group=self.mp_group)
        norm = tot.sqrt()
        if self.clip > 0:
            coef = torch.clamp(self.clip / (norm + 1e-6), max=1.0)
            for g in grads:
                g.mul_(coef.to(g.dtype))
        self.opt.step()
        return True, float(norm), None

    def state_dict(self):
        return self.opt.state_dict()

    def load_state_dict(self, sd):
        self.opt.load_state_dict(sd)

    def reload_model_params(self):
        for p, host in self.opt.cpu_copy.items():
            host.copy_(p.detach().float().cpu().reshape(host.shape))
        for p, m in self.opt.gpu_master.items():
            m.copy_(p.detach().float())
