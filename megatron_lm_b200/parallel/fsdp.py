"""Fully sharded data parallelism (ZeRO-1/2/3) over the data-parallel group, with its own sharded AdamW.

Reference: megatron/core/distributed/custom_fsdp/fully_sharded_data_parallel.py (``FullyShardedDataParallel``
:45, hooks :308-650) and custom_fsdp/param_and_grad_buffer.py (``DataParallelBuffer`` :630,
``AllGatherPipeline`` :2186, ``GradReducePipeline`` :1872), strategies ``no_shard`` / ``optim`` /
``optim_grads`` / ``optim_grads_params`` (distributed_data_parallel_config.py:120).

Design.  Parameters are grouped into *units* (one per module of the listed unit classes, plus a root
unit for the rest).  Each unit is one flat buffer, padded so that every rank owns an equal contiguous
1/dp slice; a rank keeps persistently only its slice of the weights (``optim_grads_params``), of the
fp32 gradient accumulator, and of the optimizer state.

* forward : unit weights are all-gathered into a transient full buffer just before the unit runs (the
  next unit's gather is already in flight) and dropped right after;
* backward: gathered again, gradients land in a transient fp32 full buffer through ``param.main_grad``
  (the ops of this library write there directly); when the last parameter of the unit has signalled,
  the buffer is reduce-scattered into the rank's fp32 slice and both transients are dropped;
* step    : ``ShardedAdam`` clips by the global norm and updates the slices in one launch per unit.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Type

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config import DistributedDataParallelConfig, TransformerConfig
from ..ops import optim as kops
from . import state

_STRATEGIES = ("no_shard", "optim", "optim_grads", "optim_grads_params")


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class _Unit:
    def __init__(self, name: str, params: List[nn.Parameter], group, strategy: str, grad_dtype):
        self.name, self.params, self.group, self.strategy = name, params, group, strategy
        self.dp = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.dtype = params[0].dtype
        self.device = params[0].device
        self.grad_dtype = grad_dtype
        self.offsets, off = [], 0
        for p in params:
            self.offsets.append(off)
            off = _align(off + p.numel(), 8)
        self.total = _align(max(off, 1), self.dp * 128)
        self.shard_len = self.total // self.dp
        lo = self.rank * self.shard_len
        self.lo, self.hi = lo, lo + self.shard_len
        self.shard_params = self.strategy == "optim_grads_params" and self.dp > 1
        self.shard_grads = self.strategy in ("optim_grads", "optim_grads_params") and self.dp > 1
        full = torch.zeros(self.total, dtype=self.dtype, device=self.device)
        for p, o in zip(params, self.offsets):
            full[o:o + p.numel()].copy_(p.data.reshape(-1))
        self.param_shard = full[lo:self.hi].clone()
        self.full_param: Optional[torch.Tensor] = None     # persistent tensor; its storage is emptied on release
        self.gathered = True
        self.full_grad: Optional[torch.Tensor] = None
        self.grad_shard = torch.zeros(self.shard_len, dtype=grad_dtype, device=self.device)
        self._empty = torch.empty(0, dtype=self.dtype, device=self.device)
        self.gather_handle = None
        self.pending = 0
        self.reduced = False
        self.shapes = [p.shape for p in params]
        self._install(full)
        if self.shard_params:
            self.release_params()
        if not self.shard_grads:
            self.full_grad = torch.zeros(self.total, dtype=grad_dtype, device=self.device)
            self._point_grads()

    # -- parameter views ------------------------------------------------------------
    def _install(self, full):
        self.full_param = full
        for p, o, shp in zip(self.params, self.offsets, self.shapes):
            p.data = full[o:o + shp.numel()].view(shp)

    def start_gather(self, async_op: bool = False):
        if not self.shard_params or self.gathered or self.gather_handle is not None:
            return
        # parameters stay views of the same storage (autograd keeps their shapes); only its bytes come and go
        full = self.full_param
        full.untyped_storage().resize_(self.total * full.element_size())
        if self.device.type == "cuda":
            h = dist.all_gather_into_tensor(full, self.param_shard, group=self.group, async_op=async_op)
        else:
            parts = list(full.chunk(self.dp))
            h = dist.all_gather(parts, self.param_shard, group=self.group, async_op=async_op)
        self.gather_handle = (full, h if async_op else None)

    def finish_gather(self):
        if not self.shard_params or self.gathered:
            return
        if self.gather_handle is None:
            self.start_gather(False)
        full, h = self.gather_handle
        if h is not None:
            h.wait()
        self.gather_handle = None
        self.gathered = True

    def release_params(self):
        if not self.shard_params or not self.gathered:
            return
        self.full_param.untyped_storage().resize_(0)
        self.gathered = False

    # -- gradients --------------------------------------------------------------------
    def _point_grads(self):
        for p, o, shp in zip(self.params, self.offsets, self.shapes):
            p.main_grad = self.full_grad[o:o + shp.numel()].view(shp)

    def prepare_backward(self):
        self.finish_gather()
        if self.shard_grads and self.full_grad is None:
            self.full_grad = torch.zeros(self.total, dtype=self.grad_dtype, device=self.device)
            self._point_grads()
        if self.pending <= 0:
            self.pending = sum(getattr(p, "expected_grad_signals", 1) for p in self.params if p.requires_grad)
            self.reduced = False

    def reduce_grads(self, scale: float):
        """Full gradient buffer -> this rank's slice (summed over ranks and scaled)."""
        if self.full_grad is None:
            return
        g = self.full_grad
        if scale != 1.0:
            g.mul_(scale)
        if self.dp > 1:
            if self.strategy == "no_shard":
                dist.all_reduce(g, group=self.group)
                self.grad_shard.copy_(g[self.lo:self.hi])
            else:
                tmp = torch.empty(self.shard_len, dtype=g.dtype, device=g.device)
                if g.is_cuda:
                    dist.reduce_scatter_tensor(tmp, g, group=self.group)
                else:
                    dist.all_reduce(g, group=self.group)
                    tmp.copy_(g[self.lo:self.hi])
                if self.shard_grads:
                    self.grad_shard.add_(tmp)
                else:
                    self.grad_shard.copy_(tmp)
        else:
            self.grad_shard.copy_(g)
        self.reduced = True
        if self.shard_grads:
            self.full_grad = None
            for p in self.params:
                p.main_grad = None

    def refresh_full_params(self):
        """After the optimizer wrote the weight slice: rebuild full weights where they are kept."""
        if self.shard_params:
            return
        full = self.full_param
        if self.dp > 1:
            if full.is_cuda:
                dist.all_gather_into_tensor(full, self.param_shard, group=self.group)
            else:
                dist.all_gather(list(full.chunk(self.dp)), self.param_shard, group=self.group)
        else:
            full.copy_(self.param_shard)


class FullyShardedDataParallel(nn.Module):
    def __init__(self, config: TransformerConfig, ddp_config: DistributedDataParallelConfig, module: nn.Module,
                 fsdp_unit_modules: Optional[Sequence[Type[nn.Module]]] = None, group=None,
                 disable_bucketing: bool = False):
        super().__init__()
        self.config, self.ddp_config, self.module = config, ddp_config, module
        strategy = getattr(ddp_config, "data_parallel_sharding_strategy", "optim_grads_params")
        if strategy not in _STRATEGIES:
            raise ValueError(f"unknown sharding strategy {strategy}")
        self.strategy = strategy
        if group is None and dist.is_initialized():
            group = state.get_data_parallel_group(with_context_parallel=True) if state.model_parallel_is_initialized() \
                else dist.group.WORLD
        self.group = group
        self.dp = dist.get_world_size(group) if group is not None else 1
        if fsdp_unit_modules is None:
            from ..models.transformer import TransformerLayer
            fsdp_unit_modules = (TransformerLayer,)
        grad_dtype = torch.float32 if ddp_config.grad_reduce_in_fp32 or True else None
        self.units: List[_Unit] = []
        self.unit_of: Dict[nn.Parameter, _Unit] = {}
        seen = set()
        unit_mods: List[Tuple[str, nn.Module]] = []
        for name, m in module.named_modules():
            if isinstance(m, tuple(fsdp_unit_modules)):
                ps = [p for p in m.parameters() if p.requires_grad and p not in seen]
                if ps:
                    seen.update(ps)
                    unit_mods.append((name, m))
                    self._add_unit(name, ps, grad_dtype)
        rest = [p for p in module.parameters() if p.requires_grad and p not in seen]
        self.root_unit = self._add_unit("<root>", rest, grad_dtype) if rest else None
        self.unit_mods = unit_mods
        self.is_last_microbatch = True
        self.scale = 1.0 / self.dp if (ddp_config.average_in_collective or True) else 1.0
        self.order: List[_Unit] = []
        self._install_hooks()

    def _add_unit(self, name, params, grad_dtype):
        by_dtype: Dict[torch.dtype, List[nn.Parameter]] = {}
        for p in params:
            by_dtype.setdefault(p.dtype, []).append(p)
        last = None
        for dt_, ps in by_dtype.items():
            u = _Unit(f"{name}:{dt_}", ps, self.group, self.strategy, grad_dtype)
            self.units.append(u)
            for p in ps:
                self.unit_of[p] = u
            last = u
        return last

    # -- hooks ----------------------------------------------------------------------
    def _units_of_module(self, m) -> List[_Unit]:
        out = []
        for p in m.parameters():
            u = self.unit_of.get(p)
            if u is not None and u not in out:
                out.append(u)
        return out

    def _install_hooks(self):
        for p, u in self.unit_of.items():
            p.grad_ready = (lambda p=p, u=u: self._on_grad_ready(p, u))

            def hook(param, u=u):
                # gradients produced by plain autograd: fold .grad into the unit's buffer
                if param.grad is not None:
                    if param.main_grad is not None:
                        param.main_grad.add_(param.grad.to(param.main_grad.dtype).view_as(param.main_grad))
                    param.grad = None
                    self._on_grad_ready(param, u)
            p.register_post_accumulate_grad_hook(hook)
        for name, m in self.unit_mods:
            units = [u for u in self.units if u.name.startswith(name + ":")]

            def pre(mod, args, units=units):
                for u in units:
                    u.finish_gather()
                    if u not in self.order:
                        self.order.append(u)
                    elif torch.is_grad_enabled() or True:
                        i = self.order.index(u)
                        if i + 1 < len(self.order):
                            self.order[i + 1].start_gather(async_op=u.device.type == "cuda")

            def post(mod, args, out, units=units):
                for u in units:
                    u.release_params()

            def bpre(mod, grad_out, units=units):
                for u in units:
                    u.prepare_backward()
                    i = self.order.index(u) if u in self.order else -1
                    if i > 0:
                        self.order[i - 1].start_gather(async_op=u.device.type == "cuda")
            m.register_forward_pre_hook(pre)
            m.register_forward_hook(post)
            m.register_full_backward_pre_hook(bpre)

    def _on_grad_ready(self, p, u: _Unit):
        if u.pending <= 0:
            u.prepare_backward()
        u.pending -= 1
        if u.pending == 0 and (u.shard_grads or self.is_last_microbatch) and u is not self.root_unit:
            u.reduce_grads(self.scale)
            u.release_params()

    # -- module API --------------------------------------------------------------------
    def forward(self, *a, **kw):
        for u in self.units:
            if not any(u.name.startswith(n + ":") for n, _ in self.unit_mods):
                u.finish_gather()                      # root parameters stay whole for the entire step
                u.prepare_backward() if torch.is_grad_enabled() else None
        return self.module(*a, **kw)

    @contextmanager
    def no_sync(self):
        old = self.is_last_microbatch
        self.is_last_microbatch = False
        try:
            yield
        finally:
            self.is_last_microbatch = old

    def start_grad_sync(self, *unused):
        pass

    def finish_grad_sync(self):
        """Reduce whatever has not been reduced by the per-unit triggers (root unit, units whose
        parameters were only partly used)."""
        for u in self.units:
            if u.full_grad is not None and not u.reduced:
                u.reduce_grads(self.scale)
            u.pending = 0
            if u.shard_params:
                u.release_params()

    def start_param_sync(self, *unused, force_sync: bool = False, force_dispatch: bool = False):
        for u in self.units:
            u.refresh_full_params()

    def zero_grad_buffer(self):
        for u in self.units:
            u.grad_shard.zero_()
            u.reduced = False
            u.pending = 0
            if u.full_grad is not None:
                u.full_grad.zero_()

    def scale_gradients(self, factor: float):
        for u in self.units:
            u.grad_shard.mul_(factor)

    def broadcast_params(self):
        for u in self.units:
            u.finish_gather()
            if self.dp > 1:
                dist.broadcast(u.full_param, src=dist.get_global_rank(self.group, 0), group=self.group)
                u.param_shard.copy_(u.full_param[u.lo:u.hi])
            u.release_params()

    def gathered_parameters(self):
        """Context manager: every unit whole (for checkpointing or evaluation outside the hooks)."""
        fsdp = self

        class _Ctx:
            def __enter__(self_inner):
                for u in fsdp.units:
                    u.finish_gather()

            def __exit__(self_inner, *exc):
                for u in fsdp.units:
                    u.release_params()
        return _Ctx()

    def state_dict(self, *a, **kw):
        with self.gathered_parameters():
            return {k: v.clone() for k, v in self.module.state_dict(*a, **kw).items()}

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self._modules["module"], name)


class ShardedAdam:
    """AdamW on the rank-local slices of an FSDP model: fp32 master weights and moments, global-norm
    clipping across data- and model-parallel ranks, one fused launch per unit."""

    def __init__(self, fsdp_models: Sequence[FullyShardedDataParallel], lr: float = 1e-3, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01, clip_grad: float = 0.0, model_parallel_group=None):
        self.models = list(fsdp_models)
        self.lr, self.betas, self.eps, self.wd, self.clip = lr, betas, eps, weight_decay, clip_grad
        self.mp_group = model_parallel_group
        self.step_count = 0
        self.state = []
        for m in self.models:
            for u in m.units:
                master = u.param_shard.float().clone()
                segs = []
                for p, o in zip(u.params, u.offsets):
                    a, b = max(o, u.lo), min(o + p.numel(), u.hi)
                    if a < b:
                        no_wd = p.dim() <= 1 or getattr(p, "_no_weight_decay", False)
                        segs.append((a - u.lo, b - a, 1 if no_wd else 0))
                table, n = kops.build_chunk_table(segs, u.device) if segs else (None, 0)
                self.state.append({"unit": u, "master": master, "m": torch.zeros_like(master),
                                   "v": torch.zeros_like(master), "segs": segs, "table": table, "n": n})
        self.param_groups = [{"lr": lr, "weight_decay": weight_decay, "max_lr": lr, "min_lr": 0.0, "params": []}]

    def zero_grad(self, set_to_none: bool = True):
        pass

    def scale_loss(self, loss):
        return loss

    def get_loss_scale(self) -> torch.Tensor:
        return torch.ones(1, dtype=torch.float32, device=self.state[0]["unit"].device if self.state else "cpu")

    def get_grad_norm(self) -> torch.Tensor:
        dev = self.state[0]["unit"].device
        tot = torch.zeros(1, dtype=torch.float32, device=dev)
        for st in self.state:
            u = st["unit"]
            # replicated parameters would be counted once per model-parallel rank; only rank 0 of the TP group counts them
            tp_rank0 = (not state.model_parallel_is_initialized()) or state.get_tensor_model_parallel_rank() == 0
            for (s, n, _), p in zip(st["segs"], self._seg_params(st)):
                if getattr(p, "tensor_model_parallel", False) or tp_rank0:
                    kops.sum_squares(u.grad_shard[s:s + n], tot, accumulate=True)
        for m in self.models[:1]:
            if m.group is not None and m.dp > 1:
                dist.all_reduce(tot, group=m.group)
        if self.mp_group is not None:
            dist.all_reduce(tot, group=self.mp_group)
        return tot.sqrt()

    def _seg_params(self, st):
        u = st["unit"]
        out = []
        for p, o in zip(u.params, u.offsets):
            if max(o, u.lo) < min(o + p.numel(), u.hi):
                out.append(p)
        return out

    def step(self):
        for m in self.models:
            m.finish_grad_sync()
        self.step_count += 1
        lr = self.param_groups[0]["lr"]
        norm = self.get_grad_norm()
        scale = None
        if self.clip > 0:
            scale = torch.clamp(self.clip / (norm + 1e-6), max=1.0).float()
        for st in self.state:
            if not st["segs"]:
                continue
            u = st["unit"]
            kops.adam_step(st["master"], st["m"], st["v"], u.grad_shard, table=st["table"], nchunks=st["n"],
                           lrs=[lr, lr], wds=[self.param_groups[0]["weight_decay"], 0.0], beta1=self.betas[0],
                           beta2=self.betas[1], eps=self.eps, step=self.step_count,
                           p_lp=None if u.param_shard.dtype == torch.float32 else u.param_shard, grad_scale=scale,
                           segments=st["segs"])
            if u.param_shard.dtype == torch.float32:
                u.param_shard.copy_(st["master"])
        for m in self.models:
            m.start_param_sync()
        return True, float(norm) if not norm.is_cuda else norm, None

    def state_dict(self):
        return {"step": self.step_count, "shards": [{k: st[k] for k in ("master", "m", "v")} for st in self.state]}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for st, s in zip(self.state, sd["shards"]):
            for k in ("master", "m", "v"):
                st[k].copy_(s[k])
            u = st["unit"]
            u.param_shard.copy_(st["master"].to(u.param_shard.dtype))
        for m in self.models:
            m.start_param_sync()


class TorchFullyShardedDataParallel(nn.Module):
    """Wrapper around ``torch.distributed.fsdp.fully_shard`` (FSDP2) with the DDP-like method surface the
    training loop expects (reference: megatron/core/distributed/torch_fully_sharded_data_parallel.py:36)."""

    def __init__(self, config, ddp_config, module, sub_modules_to_wrap=None, group=None):
        super().__init__()
        from torch.distributed.fsdp import fully_shard
        self.module = module
        if sub_modules_to_wrap is None:
            from ..models.transformer import TransformerLayer
            sub_modules_to_wrap = (TransformerLayer,)
        kw = {}
        if group is not None:
            from torch.distributed.device_mesh import DeviceMesh
            kw["mesh"] = DeviceMesh.from_group(group, "cuda" if torch.cuda.is_available() else "cpu")
        if not getattr(ddp_config, "torch_fsdp2_reshard_after_forward", True):
            kw["reshard_after_forward"] = False           # keep the gathered parameters until backward (more memory, no re-gather)
        for m in module.modules():
            if isinstance(m, tuple(sub_modules_to_wrap)):
                fully_shard(m, **kw)
        fully_shard(module, **kw)

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    @contextmanager
    def no_sync(self):
        self.module.set_requires_gradient_sync(False)
        try:
            yield
        finally:
            self.module.set_requires_gradient_sync(True)

    def start_grad_sync(self, *a): pass
    def finish_grad_sync(self): pass
    def start_param_sync(self, *a, **kw): pass
    def zero_grad_buffer(self): pass
    def scale_gradients(self, factor): 
        for p in self.module.parameters():
            if p.grad is not None:
                p.grad.mul_(factor)
    def broadcast_params(self): pass


class TorchOptimizerAdapter:
    """A ``torch.optim`` optimizer behind the method surface the training loop uses (``step`` returning
    ``(update_successful, grad_norm, num_zeros)``, ``scale_loss``, ``get_loss_scale``, ``param_groups`` written by
    the scheduler).  Used with torch FSDP2, whose parameters are DTensors that the flat-buffer optimizers of this
    library do not own."""

    def __init__(self, params, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 clip_grad: float = 0.0, optimizer: str = "adam", momentum: float = 0.0):
        params = [p for p in params if p.requires_grad]
        decay = [p for p in params if p.dim() > 1]
        no_decay = [p for p in params if p.dim() <= 1]
        groups = [dict(params=decay, weight_decay=weight_decay, wd_mult=1.0, lr_mult=1.0, max_lr=lr, min_lr=0.0),
                  dict(params=no_decay, weight_decay=0.0, wd_mult=0.0, lr_mult=1.0, max_lr=lr, min_lr=0.0)]
        groups = [g for g in groups if g["params"]]
        if optimizer == "adam":
            self.opt = torch.optim.AdamW(groups, lr=lr, betas=betas, eps=eps)
        elif optimizer == "sgd":
            self.opt = torch.optim.SGD(groups, lr=lr, momentum=momentum)
        else:
            raise ValueError(f"unknown optimizer {optimizer}")
        self.clip = clip_grad
        self.params = params

    @property
    def param_groups(self):
        return self.opt.param_groups

    def zero_grad(self, set_to_none: bool = True):
        self.opt.zero_grad(set_to_none=set_to_none)

    def scale_loss(self, loss):
        return loss

    def get_loss_scale(self) -> torch.Tensor:
        return torch.ones(1, dtype=torch.float32)

    def step(self):
        for g in self.opt.param_groups:                 # the scheduler writes one decay value; groups scale it
            g["weight_decay"] = g["weight_decay"] * g.get("wd_mult", 1.0) if g.get("wd_mult", 1.0) == 0.0 \
                else g["weight_decay"]
        with_grad = [p for p in self.params if p.grad is not None]
        norm = torch.nn.utils.clip_grad_norm_(with_grad, self.clip if self.clip > 0 else float("inf"))
        if hasattr(norm, "full_tensor"):
            norm = norm.full_tensor()
        self.opt.step()
        return True, float(norm), None

    def materialize_state(self):
        """Create the optimizer's per-parameter slots (torch builds them at the first step) without moving the
        weights: one step with zero gradients at learning rate 0.  Needed before a checkpoint's state is copied in."""
        saved = [(g["lr"], g["weight_decay"]) for g in self.opt.param_groups]
        for g in self.opt.param_groups:
            g["lr"], g["weight_decay"] = 0.0, 0.0
        for p in self.params:
            p.grad = torch.zeros_like(p)
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        for g, (lr, wd) in zip(self.opt.param_groups, saved):
            g["lr"], g["weight_decay"] = lr, wd

    def state_dict(self):
        return self.opt.state_dict()

    def load_state_dict(self, sd):
        self.opt.load_state_dict(sd)

    def reload_model_params(self):
        pass
