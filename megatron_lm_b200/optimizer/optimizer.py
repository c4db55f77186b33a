"""Mixed-precision optimizer over the flat DDP buffers (plain and ZeRO-1 sharded).

Step order matches the reference (megatron/core/optimizer/optimizer.py:392-580,
distrib_optimizer.py:2030-2269, clip_grads.py:51-178): gradients ready in the
buffer -> global L2 norm over model-parallel (+ DP shard) ranks -> overflow
check -> clip coefficient ``clip / (norm + 1e-6)`` -> AdamW on fp32 master
weights -> low-precision copy back -> (distributed) parameter all-gather.

What is different: master weights, ``exp_avg`` and ``exp_avg_sq`` are flat fp32
tensors laid out exactly like this rank's slice of each gradient buffer, so one
kernel launch per buffer performs unscale + clip + Adam + the bf16 write-back
into the parameter buffer, driven by a chunk table that carries each
parameter's hyper-parameter group.  The clip coefficient and the overflow flag
stay on the device; the host never synchronises inside ``step``.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..config import OptimizerConfig
from ..ops import optim as K
from ..parallel import state
from ..parallel.ddp import DistributedDataParallel, ParamAndGradBuffer
from .grad_scaler import ConstantGradScaler, DynamicGradScaler


def param_group_key(name: str, p: torch.Tensor, no_wd_cond: Optional[Callable] = None,
                    scale_lr_cond: Optional[Callable] = None, lr_mult: float = 1.0) -> Tuple[float, float]:
    """(wd_mult, lr_mult): biases and 1-d parameters take no weight decay
    (reference: optimizer/__init__.py:48-165)."""
    if no_wd_cond is not None:
        no_wd = no_wd_cond(name, p)
    else:
        no_wd = name.endswith(".bias") or p.dim() == 1
    scale = scale_lr_cond(name, p) if scale_lr_cond is not None else False
    return (0.0 if no_wd else 1.0, lr_mult if scale else 1.0)


class _BufferState:
    """Optimizer state for this rank's part of one buffer."""

    def __init__(self, buf: ParamAndGradBuffer, names: Dict[torch.Tensor, str], group_of: Callable, sharded: bool,
                 count_in_norm: Callable):
        self.buf, self.sharded = buf, sharded
        # flat local index space: concatenation of this rank's slice of every bucket
        self.ranges: List[Tuple[int, int, int]] = []          # (buffer start, buffer end, local start)
        local = 0
        for b in buf.buckets:
            s, e = buf.shard_range(b) if sharded else (b.start, b.end)
            self.ranges.append((s, e, local))
            local += e - s
        self.local_numel = local
        dev = buf.param_data.device
        self.contiguous = len(self.ranges) == 1 or not sharded
        if self.contiguous:
            s0 = self.ranges[0][0]
            e0 = self.ranges[-1][1]
            self.ranges = [(s0, e0, 0)]
            self.local_numel = e0 - s0
        self.master = torch.zeros(self.local_numel, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        # per-parameter pieces inside the local space
        self.pieces: List[dict] = []
        segments, excluded = [], []
        for p in buf.params:
            ps, pe, _ = buf.param_index_map[p]
            for (s, e, l0) in self.ranges:
                lo, hi = max(ps, s), min(pe, e)
                if lo >= hi:
                    continue
                piece = dict(param=p, name=names[p], buf_start=lo, local_start=l0 + (lo - s), numel=hi - lo,
                             param_start=lo - ps, group=group_of(names[p], p))
                self.pieces.append(piece)
                segments.append((piece["local_start"], piece["numel"], piece["group"]))
                if not count_in_norm(p):
                    excluded.append((piece["local_start"], piece["numel"]))
        self.segments = segments
        self.excluded = excluded
        self.nchunks = len(segments)
        # one chunk table per contiguous range, addressed relative to the range start
        self.range_tables = {}
        for (s, e, l0) in self.ranges:
            segs = [(ls - l0, n, g) for (ls, n, g) in segments if l0 <= ls < l0 + (e - s)]
            table, nchunks = K.build_chunk_table(segs, dev) if segs else (None, 0)
            self.range_tables[(s, e)] = (table, nchunks, segs)
        self.reload_master_from_params()

    def views(self, flat: torch.Tensor):
        """(buffer slice, local slice) pairs for copying between a full buffer and local space."""
        for (s, e, l0) in self.ranges:
            yield flat[s:e], l0, e - s

    def reload_master_from_params(self):
        for (s, e, l0) in self.ranges:
            self.master[l0:l0 + e - s].copy_(self.buf.param_data[s:e])


class MixedPrecisionOptimizer:
    """AdamW/SGD with fp32 master weights over DDP buffers; ``use_distributed_optimizer``
    shards master weights and moments 1/dp per rank (ZeRO-1)."""

    def __init__(self, config: OptimizerConfig, model_chunks: Sequence[DistributedDataParallel],
                 no_weight_decay_cond=None, scale_lr_cond=None, lr_mult: float = 1.0, expert: Optional[bool] = None):
        self.config = config
        self.model_chunks = list(model_chunks)
        self.sharded = config.use_distributed_optimizer
        self.expert_only = expert is True
        self.step_count = 0
        self.groups: List[Tuple[float, float]] = []

        def group_of(name, p):
            key = param_group_key(name, p, no_weight_decay_cond, scale_lr_cond, lr_mult)
            if key not in self.groups:
                self.groups.append(key)
            return self.groups.index(key)

        tp_rank = state.get_tensor_model_parallel_rank() if state.model_parallel_is_initialized() else 0

        def count_in_norm(p):
            # shared copies and tensor-parallel duplicates are counted once
            if getattr(p, "shared", False):
                return False
            return getattr(p, "tensor_model_parallel", False) or tp_rank == 0

        self.states: List[_BufferState] = []
        for chunk in self.model_chunks:
            names = {p: n for n, p in chunk.module.named_parameters()}
            bufs = []
            if expert is None or expert is False:
                bufs += chunk.buffers
            if expert is None or expert is True:
                bufs += chunk.expert_buffers
            for buf in bufs:
                self.states.append(_BufferState(buf, names, group_of, self.sharded and buf.dp_size > 1, count_in_norm))
        self.lr = config.lr or 0.0
        self.weight_decay = config.weight_decay
        dev = self.states[0].master.device if self.states else torch.device("cpu")
        self.device = dev
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._excl_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_scale = torch.ones(1, dtype=torch.float32, device=dev)
        self.found_inf = torch.zeros(1, dtype=torch.float32, device=dev)
        if config.fp16:
            self.grad_scaler = (ConstantGradScaler(config.loss_scale) if config.loss_scale else
                                DynamicGradScaler(config.initial_loss_scale, config.min_loss_scale, 2.0, 0.5,
                                                  config.loss_scale_window, config.hysteresis))
        elif config.loss_scale:
            self.grad_scaler = ConstantGradScaler(config.loss_scale)
        else:
            self.grad_scaler = None
        # the scheduler writes these
        self.param_groups = [dict(lr=self.lr, weight_decay=self.weight_decay, wd_mult=w, lr_mult=l,
                                  max_lr=config.lr, min_lr=config.min_lr)
                             for (w, l) in (self.groups or [(1.0, 1.0)])]

    # -- loss scale -------------------------------------------------------------
    def get_loss_scale(self) -> torch.Tensor:
        if self.grad_scaler is None:
            return torch.ones(1, dtype=torch.float32, device=self.device)
        return torch.tensor([self.grad_scaler.scale], dtype=torch.float32, device=self.device)

    def scale_loss(self, loss):
        return loss if self.grad_scaler is None else loss * self.grad_scaler.scale

    def zero_grad(self, set_to_none: bool = True):
        for chunk in self.model_chunks:
            chunk.zero_grad_buffer()

    # -- norm ---------------------------------------------------------------------
    def _stats_group(self):
        if not (state.model_parallel_is_initialized() and dist.is_initialized()):
            return None
        return None if state.get_world_size() == 1 else "stats"

    def compute_grad_norm_sq(self) -> torch.Tensor:
        """Sum of squares of this rank's (unscaled) gradient pieces, then reduced over the
        model-parallel group and, when sharded, over the data-parallel group."""
        self._norm_sq.zero_()
        self._excl_sq.zero_()
        for st in self.states:
            for (s, e, _l0) in st.ranges:
                K.sum_squares(st.buf.grad_data[s:e], self._norm_sq, accumulate=True)
            for (l0, n) in st.excluded:
                # excluded pieces are small (norm weights on tp_rank > 0, tied copies)
                for (s, e, base) in st.ranges:
                    if base <= l0 < base + (e - s):
                        K.sum_squares(st.buf.grad_data[s + (l0 - base): s + (l0 - base) + n], self._excl_sq,
                                      accumulate=True)
        total = self._norm_sq - self._excl_sq
        if state.model_parallel_is_initialized() and dist.is_initialized():
            if self.expert_only:
                # expert parameters differ across expert-parallel ranks: their norm is summed over the expert
                # model-parallel group (tp x ep x pp), and over the expert data-parallel group when sharded
                # (reference: optimizer/clip_grads.py with the tp-ep-pp group of expert optimizers)
                if state.get_group_size("tp_ep_pp") > 1:
                    dist.all_reduce(total, group=state.get_expert_tensor_model_pipeline_parallel_group())
                if self.sharded and state.get_expert_data_parallel_world_size() > 1:
                    dist.all_reduce(total, group=state.get_expert_data_parallel_group())
            else:
                if state.get_group_size("mp") > 1:
                    dist.all_reduce(total, group=state.get_model_parallel_group())
                # shards live inside one optimizer instance (the whole data-parallel group unless several
                # instances were asked for): other instances hold copies of the same shards
                if self.sharded and state.get_data_parallel_world_size(with_context_parallel=True,
                                                                       partial_data_parallel=True) > 1:
                    dist.all_reduce(total, group=state.get_data_parallel_group(with_context_parallel=True,
                                                                               partial_data_parallel=True))
        return total

    # -- step ---------------------------------------------------------------------
    def prepare_grads(self) -> torch.Tensor:
        """Compute the global grad norm and leave clip coefficient / overflow flag on device."""
        inv_scale = 1.0 if self.grad_scaler is None else 1.0 / self.grad_scaler.scale
        norm = torch.sqrt(self.compute_grad_norm_sq()) * inv_scale
        finite = torch.isfinite(norm)
        self.found_inf.copy_((~finite).float())
        if self.config.clip_grad > 0.0:
            coef = torch.clamp(self.config.clip_grad / (norm + 1.0e-6), max=1.0)
        else:
            coef = torch.ones_like(norm)
        self.grad_scale.copy_(torch.where(finite, coef * inv_scale, torch.zeros_like(coef)))
        return norm

    def step_with_ready_grads(self) -> None:
        cfg = self.config
        self.step_count += 1
        lrs = [g["lr"] * g["lr_mult"] for g in self.param_groups]
        wds = [g["weight_decay"] * g["wd_mult"] for g in self.param_groups]
        for st in self.states:
            if st.nchunks == 0:
                continue
            buf = st.buf
            for (s, e, l0) in st.ranges:
                n = e - s
                # the chunk table addresses local space; with one contiguous range per buffer the
                # gradient / parameter slices line up with it directly
                g = buf.grad_data[s:e]
                lp = buf.param_data[s:e] if buf.param_dtype != torch.float32 else None
                table, nchunks, segs = st.range_tables[(s, e)]
                if nchunks == 0:
                    continue
                master = st.master[l0:l0 + n]
                if cfg.optimizer == "adam":
                    peer_lp = None
                    if getattr(buf, "peer", None) is not None and lp is not None:
                        peer_lp = [base + 2 * s for q, base in enumerate(buf.peer["param"]) if q != buf.dp_rank]
                    K.adam_step(master, st.exp_avg[l0:l0 + n], st.exp_avg_sq[l0:l0 + n], g, table=table,
                                nchunks=nchunks, lrs=lrs, wds=wds, beta1=cfg.adam_beta1, beta2=cfg.adam_beta2,
                                eps=cfg.adam_eps, step=self.step_count, p_lp=lp, grad_scale=self.grad_scale,
                                skip=self.found_inf, segments=segs, peer_lp=peer_lp)
                else:
                    K.sgd_step(master, st.exp_avg[l0:l0 + n], g, table=table, nchunks=nchunks, lrs=lrs, wds=wds,
                               momentum=cfg.sgd_momentum, first_step=self.step_count == 1, p_lp=lp,
                               grad_scale=self.grad_scale, skip=self.found_inf, segments=segs)
                if lp is None:
                    buf.param_data[s:e].copy_(master)
        for st in self.states:
            if getattr(st.buf, "peer", None) is not None:
                st.buf.peer_barrier()            # every rank's pushed weights have landed before the next forward
        from ..ops.fp8 import weights_updated
        weights_updated()                        # cached FP8 copies of the weights are out of date
        mine = {id(st.buf) for st in self.states}
        for chunk in self.model_chunks:
            bufs = [b for b in chunk.buffers + chunk.expert_buffers if id(b) in mine]
            chunk.mark_params_updated(bufs)
            chunk.start_param_sync(buffers=bufs)

    def step(self):
        """Returns (update_successful, grad_norm, num_zeros_in_grad).  ``update_successful`` is
        only materialised on the host when loss scaling is dynamic (fp16); otherwise True."""
        norm = self.prepare_grads()
        zeros = None
        if self.config.log_num_zeros_in_grad:
            zeros = sum(K.count_zeros(st.buf.grad_data[s:e]) for st in self.states for (s, e, _) in st.ranges)
            if dist.is_initialized() and state.model_parallel_is_initialized():
                dist.all_reduce(zeros, group=state.get_model_parallel_group())
        ok = True
        if isinstance(self.grad_scaler, DynamicGradScaler):
            found = bool(self.found_inf.item() != 0.0)
            self.grad_scaler.update(found)
            ok = not found
        if ok:
            self.step_with_ready_grads()
        return ok, norm, zeros

    # -- (de)serialisation ------------------------------------------------------
    def state_dict(self):
        return {
            "step": self.step_count,
            "param_groups": [dict(g) for g in self.param_groups],
            "grad_scaler": None if self.grad_scaler is None else self.grad_scaler.state_dict(),
            "state": [dict(master=st.master.detach().cpu(), exp_avg=st.exp_avg.detach().cpu(),
                           exp_avg_sq=st.exp_avg_sq.detach().cpu()) for st in self.states],
        }

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for g, s in zip(self.param_groups, sd["param_groups"]):
            g.update(s)
        if self.grad_scaler is not None and sd.get("grad_scaler") is not None:
            self.grad_scaler.load_state_dict(sd["grad_scaler"])
        for st, s in zip(self.states, sd["state"]):
            st.master.copy_(s["master"])
            st.exp_avg.copy_(s["exp_avg"])
            st.exp_avg_sq.copy_(s["exp_avg_sq"])

    def reload_model_params(self):
        for st in self.states:
            st.reload_master_from_params()

    def local_state_tensors(self) -> List[torch.Tensor]:
        """Flat fp32 tensors (master, exp_avg, exp_avg_sq per buffer): the stripe members of the
        erasure-coded in-memory checkpoint."""
        out = []
        for st in self.states:
            out += [st.master, st.exp_avg, st.exp_avg_sq]
        return out


class ChainedOptimizer:
    """Several optimizers stepped as one (dense + expert), sharing the clip coefficient
    (reference: optimizer.py:1031)."""

    def __init__(self, optimizers: Sequence[MixedPrecisionOptimizer]):
        self.chained_optimizers = list(optimizers)

    @property
    def param_groups(self):
        return [g for o in self.chained_optimizers for g in o.param_groups]

    def zero_grad(self, set_to_none: bool = True):
        for o in self.chained_optimizers:
            o.zero_grad(set_to_none)

    def get_loss_scale(self):
        return self.chained_optimizers[0].get_loss_scale()

    def scale_loss(self, loss):
        return self.chained_optimizers[0].scale_loss(loss)

    def step(self):
        sq = None
        for o in self.chained_optimizers:
            s = o.compute_grad_norm_sq()
            sq = s.clone() if sq is None else sq + s
        first = self.chained_optimizers[0]
        inv = 1.0 if first.grad_scaler is None else 1.0 / first.grad_scaler.scale
        norm = torch.sqrt(sq) * inv
        finite = torch.isfinite(norm)
        clip = first.config.clip_grad
        coef = torch.clamp(clip / (norm + 1e-6), max=1.0) if clip > 0 else torch.ones_like(norm)
        ok = True
        if isinstance(first.grad_scaler, DynamicGradScaler):
            found = bool((~finite).item())
            for o in self.chained_optimizers:
                if o.grad_scaler is not None:
                    o.grad_scaler.update(found)
            ok = not found
        for o in self.chained_optimizers:
            o.found_inf.copy_((~finite).float())
            o.grad_scale.copy_(torch.where(finite, coef * inv, torch.zeros_like(coef)))
            if ok:
                o.step_with_ready_grads()
        return ok, norm, None

    def state_dict(self):
        return [o.state_dict() for o in self.chained_optimizers]

    def load_state_dict(self, sds):
        for o, sd in zip(self.chained_optimizers, sds):
            o.load_state_dict(sd)

    def reload_model_params(self):
        for o in self.chained_optimizers:
            o.reload_model_params()

    def local_state_tensors(self):
        return [t for o in self.chained_optimizers for t in o.local_state_tensors()]


def get_megatron_optimizer(config: OptimizerConfig, model_chunks, no_weight_decay_cond=None, scale_lr_cond=None,
                           lr_mult: float = 1.0):
    """Dense optimizer, plus a separate expert optimizer when the model has expert-parallel
    parameters (they reduce over a different data-parallel group)
    (reference: optimizer/__init__.py:479-757)."""
    model_chunks = list(model_chunks)
    has_dense = any(c.buffers for c in model_chunks)
    has_expert = any(c.expert_buffers for c in model_chunks)
    opts = []
    if has_dense:
        opts.append(MixedPrecisionOptimizer(config, model_chunks, no_weight_decay_cond, scale_lr_cond, lr_mult,
                                            expert=False))
    if has_expert:
        opts.append(MixedPrecisionOptimizer(config, model_chunks, no_weight_decay_cond, scale_lr_cond, lr_mult,
                                            expert=True))
    if len(opts) == 1:
        return opts[0]
    return ChainedOptimizer(opts)
