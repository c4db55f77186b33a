"""Model/optimizer construction and the training step.

Mirrors the reference harness (megatron/training/training.py: ``get_model`` :1014,
``setup_model_and_optimizer`` :1223, ``train_step`` :1381, loss averaging :1484-1518,
callback installation :2134-2152) but as a library usable without global args: the pieces
take explicit config objects and the step is a plain function.
"""
from __future__ import annotations

import contextlib
import time
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig
from ..optimizer import OptimizerParamScheduler, get_megatron_optimizer
from ..parallel import state
from ..parallel.ddp import DistributedDataParallel
from ..parallel.finalize_model_grads import finalize_model_grads
from ..parallel.schedules import get_forward_backward_func


def get_model(model_provider: Callable, config: TransformerConfig, ddp_config: Optional[DistributedDataParallelConfig]
              = None, wrap_with_ddp: bool = True) -> List[torch.nn.Module]:
    """Build one model chunk per virtual pipeline stage and wrap each in the DDP buffers.

    ``model_provider(pre_process, post_process, vp_stage=None)`` returns a module."""
    init = state.model_parallel_is_initialized()
    pp = state.get_pipeline_model_parallel_world_size() if init else 1
    vpp = state.get_virtual_pipeline_model_parallel_world_size() if init else None
    if init and torch.cuda.is_available():
        # pipeline transfers and data-parallel reductions are long-running kernels on other streams: let the
        # persistent GEMM hand its tiles to whichever blocks are running instead of to block numbers
        from ..ops.gemm import set_dynamic_schedule
        set_dynamic_schedule(pp > 1 or state.get_data_parallel_world_size(with_context_parallel=True) > 1)
    chunks = []
    if pp > 1 and vpp is not None and vpp > 1:
        for i in range(vpp):
            state.set_virtual_pipeline_model_parallel_rank(i)
            pre = state.is_pipeline_first_stage(ignore_virtual=False, vp_stage=i)
            post = state.is_pipeline_last_stage(ignore_virtual=False, vp_stage=i)
            chunks.append(model_provider(pre_process=pre, post_process=post, vp_stage=i))
        state.set_virtual_pipeline_model_parallel_rank(0)
    else:
        pre = state.is_pipeline_first_stage() if init else True
        post = state.is_pipeline_last_stage() if init else True
        chunks.append(model_provider(pre_process=pre, post_process=post))
    for m in chunks:
        for p in m.parameters():
            if not hasattr(p, "tensor_model_parallel"):
                p.tensor_model_parallel = False
    if not wrap_with_ddp:
        return chunks
    ddp_config = ddp_config or DistributedDataParallelConfig()
    wrapped = []
    if getattr(ddp_config, "use_custom_fsdp", False) or getattr(ddp_config, "use_torch_fsdp2", False):
        # sharded data parallelism (ZeRO-1/2/3 units or torch FSDP2) instead of the replicated buffers
        from ..parallel.fsdp import FullyShardedDataParallel, TorchFullyShardedDataParallel
        cls = FullyShardedDataParallel if getattr(ddp_config, "use_custom_fsdp", False) else TorchFullyShardedDataParallel
        return [cls(config, ddp_config, m) for m in chunks]
    for i, m in enumerate(chunks):
        # bucketing only helps overlap on the first chunk; later chunks sync as one bucket
        wrapped.append(DistributedDataParallel(config, ddp_config, m, disable_bucketing=(i > 0) or
                                               (not ddp_config.overlap_grad_reduce)))
    if config.__dict__.get("data_parallel_random_init", False):
        for w in wrapped:
            w.broadcast_params()
    return wrapped


def get_optimizer_param_scheduler(optimizer, *, lr: float, min_lr: float = 0.0, lr_decay_style: str = "linear",
                                  train_iters: Optional[int] = None, global_batch_size: int = 1,
                                  lr_decay_iters: Optional[int] = None, lr_warmup_iters: int = 0,
                                  lr_warmup_fraction: Optional[float] = None, lr_warmup_init: float = 0.0,
                                  weight_decay: float = 0.01, start_weight_decay: Optional[float] = None,
                                  end_weight_decay: Optional[float] = None, weight_decay_incr_style: str = "constant",
                                  lr_wsd_decay_style=None, lr_wsd_decay_iters=None, lr_decay_samples=None,
                                  lr_warmup_samples: int = 0, lr_wsd_decay_samples=None, **kw) -> OptimizerParamScheduler:
    """Schedules are stepped in samples, so iteration counts are multiplied by the global batch
    (reference: training.py:1167-1221)."""
    decay_iters = lr_decay_iters or train_iters or 1
    decay_steps = decay_iters * global_batch_size
    wd_steps = (train_iters or decay_iters) * global_batch_size
    if lr_warmup_fraction is not None:
        warm = int(lr_warmup_fraction * decay_steps)
    else:
        warm = lr_warmup_iters * global_batch_size
    # sample-based forms of the same settings (--lr-decay-samples, --lr-warmup-samples, --lr-wsd-decay-samples)
    if lr_decay_samples is not None:
        decay_steps = lr_decay_samples
    if lr_warmup_samples:
        warm = lr_warmup_samples
    wsd_steps = lr_wsd_decay_samples if lr_wsd_decay_samples is not None else \
        (lr_wsd_decay_iters * global_batch_size if lr_wsd_decay_iters else None)
    sw = weight_decay if start_weight_decay is None else start_weight_decay
    ew = weight_decay if end_weight_decay is None else end_weight_decay
    return OptimizerParamScheduler(optimizer, init_lr=lr_warmup_init, max_lr=lr, min_lr=min_lr, lr_warmup_steps=warm,
                                   lr_decay_steps=decay_steps, lr_decay_style=lr_decay_style, start_wd=sw, end_wd=ew,
                                   wd_incr_steps=wd_steps, wd_incr_style=weight_decay_incr_style,
                                   wsd_decay_steps=wsd_steps,
                                   lr_wsd_decay_style=lr_wsd_decay_style, use_checkpoint_opt_param_scheduler=False)


def build_optimizer(optimizer_config: OptimizerConfig, model, no_wd_decay_cond=None, scale_lr_cond=None,
                    lr_mult: float = 1.0, cpu_offload: bool = False, offload_fraction: float = 1.0):
    """The optimizer that fits how ``model`` is wrapped: sharded AdamW for FSDP chunks, the host-resident hybrid
    optimizer when offloading is asked for, else the flat mixed-precision (optionally ZeRO-1) optimizer."""
    from ..parallel.fsdp import FullyShardedDataParallel
    if model and isinstance(model[0], FullyShardedDataParallel):
        from ..parallel.fsdp import ShardedAdam
        if optimizer_config.optimizer != "adam":
            raise ValueError("the sharded (FSDP) data-parallel path implements AdamW only")
        mp = state.get_model_parallel_group() if state.model_parallel_is_initialized() and \
            state.get_group_size("mp") > 1 else None
        return ShardedAdam(model, lr=optimizer_config.lr or 0.0,
                           betas=(optimizer_config.adam_beta1, optimizer_config.adam_beta2),
                           eps=optimizer_config.adam_eps, weight_decay=optimizer_config.weight_decay,
                           clip_grad=optimizer_config.clip_grad or 0.0, model_parallel_group=mp)
    from ..parallel.fsdp import TorchFullyShardedDataParallel
    if model and isinstance(model[0], TorchFullyShardedDataParallel):
        from ..parallel.fsdp import TorchOptimizerAdapter
        params = [p for m in model for p in m.parameters()]
        return TorchOptimizerAdapter(params, lr=optimizer_config.lr or 0.0,
                                     betas=(optimizer_config.adam_beta1, optimizer_config.adam_beta2),
                                     eps=optimizer_config.adam_eps, weight_decay=optimizer_config.weight_decay,
                                     clip_grad=optimizer_config.clip_grad or 0.0, optimizer=optimizer_config.optimizer,
                                     momentum=optimizer_config.sgd_momentum)
    if getattr(optimizer_config, "optimizer_cpu_offload", False):
        from ..optimizer.cpu_offload import OffloadedOptimizer
        if optimizer_config.use_distributed_optimizer or optimizer_config.optimizer != "adam":
            raise ValueError("--optimizer-cpu-offload here covers AdamW without the distributed optimizer")
        mp = state.get_model_parallel_group() if state.model_parallel_is_initialized() and \
            state.get_group_size("mp") > 1 else None
        return OffloadedOptimizer([m.module for m in model], lr=optimizer_config.lr or 0.0,
                                  betas=(optimizer_config.adam_beta1, optimizer_config.adam_beta2),
                                  eps=optimizer_config.adam_eps, weight_decay=optimizer_config.weight_decay,
                                  clip_grad=optimizer_config.clip_grad or 0.0,
                                  offload_fraction=optimizer_config.optimizer_offload_fraction,
                                  model_parallel_group=mp)
    return get_megatron_optimizer(optimizer_config, model, no_wd_decay_cond, scale_lr_cond, lr_mult)


def setup_model_and_optimizer(model_provider, config: TransformerConfig, optimizer_config: OptimizerConfig,
                              ddp_config: Optional[DistributedDataParallelConfig] = None, scheduler_kwargs=None,
                              no_wd_decay_cond=None, scale_lr_cond=None, lr_mult: float = 1.0):
    model = get_model(model_provider, config, ddp_config)
    optimizer = build_optimizer(optimizer_config, model, no_wd_decay_cond, scale_lr_cond, lr_mult)
    scheduler = None
    if scheduler_kwargs is not None:
        scheduler = get_optimizer_param_scheduler(optimizer, **scheduler_kwargs)
    install_callbacks(config, model, optimizer)
    return model, optimizer, scheduler


def install_callbacks(config: TransformerConfig, model: Sequence[torch.nn.Module], optimizer) -> None:
    """Hand the schedules the hooks they call back (reference: training.py:2134-2152)."""
    if all(hasattr(m, "no_sync") for m in model):
        config.no_sync_func = [m.no_sync for m in model] if len(model) > 1 else model[0].no_sync
        config.grad_sync_func = [m.start_grad_sync for m in model] if len(model) > 1 else model[0].start_grad_sync
        config.param_sync_func = [m.start_param_sync for m in model] if len(model) > 1 else model[0].start_param_sync
    config.finalize_model_grads_func = finalize_model_grads
    config.grad_scale_func = optimizer.scale_loss if optimizer is not None else None


def train_step(forward_step_func, data_iterator, model: Sequence[torch.nn.Module], optimizer, opt_param_scheduler,
               config: TransformerConfig, *, num_microbatches: int, seq_length: int, micro_batch_size: int,
               global_batch_size: Optional[int] = None, rerun_state_machine=None):
    """One optimizer step.  Returns (loss dict, skipped_iter, grad_norm, num_zeros_in_grad)."""
    fb = get_forward_backward_func()

    def run_once():
        for m in model:
            if hasattr(m, "zero_grad_buffer"):
                m.zero_grad_buffer()
        optimizer.zero_grad()
        return fb(forward_step_func=forward_step_func, data_iterator=data_iterator, model=list(model),
                  num_microbatches=num_microbatches, seq_length=seq_length, micro_batch_size=micro_batch_size,
                  forward_only=False)

    if rerun_state_machine is None:
        losses = run_once()
    else:
        # normally one pass; a suspicious result makes every rank replay the step
        losses = []
        while rerun_state_machine.should_run_forward_backward(data_iterator):
            losses = run_once()
        if rerun_state_machine.should_checkpoint_and_exit()[0]:
            # the caller saves the state from before this step and exits: no update is applied
            return {}, 1, None, None
    ok, grad_norm, zeros = optimizer.step()
    skipped = 0 if ok else 1
    if ok and opt_param_scheduler is not None:
        dp = state.get_data_parallel_world_size() if state.model_parallel_is_initialized() else 1
        inc = global_batch_size if global_batch_size is not None else num_microbatches * micro_batch_size * dp
        opt_param_scheduler.step(increment=inc)
    return reduce_losses(losses, config), skipped, grad_norm, zeros


def reduce_losses(losses: List[dict], config) -> Dict[str, torch.Tensor]:
    """Average each reported key over microbatches and data-parallel ranks on the last stage
    (reference: training.py:1484-1518).  A value may be a scalar or a (sum, count) pair."""
    if not losses:
        return {}
    out = {}
    for key in losses[0].keys():
        vals = [d[key] for d in losses]
        if vals[0].numel() == 2:
            v = torch.stack(vals).sum(dim=0).float()
            if dist.is_initialized() and state.model_parallel_is_initialized() and \
                    state.get_data_parallel_world_size(with_context_parallel=True) > 1:
                dist.all_reduce(v, group=state.get_data_parallel_group(with_context_parallel=True))
            out[key] = v[0] / v[1].clamp(min=1)
        else:
            v = torch.stack([x.reshape(()) for x in vals]).float().mean()
            if dist.is_initialized() and state.model_parallel_is_initialized() and \
                    state.get_data_parallel_world_size(with_context_parallel=True) > 1:
                dist.all_reduce(v, group=state.get_data_parallel_group(with_context_parallel=True),
                                op=dist.ReduceOp.AVG if dist.get_backend() == "nccl" else dist.ReduceOp.SUM)
                if dist.get_backend() != "nccl":
                    v = v / state.get_data_parallel_world_size(with_context_parallel=True)
            out[key] = v
    return out


def evaluate(forward_step_func, data_iterator, model, config, *, eval_iters: int, num_microbatches: int,
             seq_length: int, micro_batch_size: int) -> Dict[str, float]:
    """Forward-only passes averaged over ``eval_iters`` (reference: training.py:2413)."""
    for m in model:
        sync = getattr(m, "force_param_sync", None)
        if sync is not None:
            sync()                       # evaluation must see this step's weights from every data-parallel rank
        m.eval()
    fb = get_forward_backward_func()
    totals: Dict[str, float] = {}
    with torch.no_grad():
        for _ in range(eval_iters):
            losses = fb(forward_step_func=forward_step_func, data_iterator=data_iterator, model=list(model),
                        num_microbatches=num_microbatches, seq_length=seq_length,
                        micro_batch_size=micro_batch_size, forward_only=True)
            for k, v in reduce_losses(losses, config).items():
                totals[k] = totals.get(k, 0.0) + float(v)
    for m in model:
        m.train()
    return {k: v / max(eval_iters, 1) for k, v in totals.items()}
