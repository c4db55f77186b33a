"""The training program: initialise, build model/optimizer/data, run the loop, log, checkpoint.

Counterpart of the reference's ``pretrain`` / ``train`` / ``training_log`` (megatron/training/
training.py:706, :2070, :1531) and ``initialize_megatron`` (initialize.py:38).  Scalar names in the
log and on TensorBoard match the reference (``lm loss``, ``iteration-time``, ``learning-rate``,
``grad-norm``, ``throughput`` in TFLOP/s/GPU by the reference's FLOP formula), so its result
parsers keep working.
"""
from __future__ import annotations

import os
import signal
import sys
import math
import time
from datetime import timedelta
from typing import Callable, Dict, Optional

import torch
import torch.distributed as dist

from ..checkpoint.ec_checkpoint import ECCheckpointManager
from ..data.tokenizer import build_tokenizer
from ..parallel import state
from ..parallel.random import model_parallel_cuda_manual_seed
from ..utils.timers import Timers
from . import checkpointing
from .arguments import (core_transformer_config_from_args, ddp_config_from_args, get_args, optimizer_config_from_args,
                        parse_args, set_args, validate_args)
from .flops import flops_from_config
from .resilience import DistributedSignalHandler, RerunStateMachine, StragglerDetector
from .training import (build_optimizer, evaluate, get_model, get_optimizer_param_scheduler, install_callbacks,
                       train_step)
from ..optimizer import get_megatron_optimizer

_TIMERS: Optional[Timers] = None
_WRITER = None


def print_rank_0(msg: str) -> None:
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(msg, flush=True)


def print_rank_last(msg: str) -> None:
    if not dist.is_initialized() or dist.get_rank() == dist.get_world_size() - 1:
        print(msg, flush=True)


def get_timers() -> Timers:
    return _TIMERS


def initialize_megatron(extra_args_provider=None, args_defaults=None, ignore_unknown_args=False, argv=None,
                        store=None):
    """Parse arguments, start torch.distributed, build the parallel groups, seed the RNG streams."""
    global _TIMERS, _WRITER
    args = parse_args(extra_args_provider, ignore_unknown_args, argv)
    if getattr(args, "yaml_cfg", None):
        from .arguments import load_yaml_args
        args = load_yaml_args(args.yaml_cfg, args)
    if getattr(args, "use_checkpoint_args", False) or getattr(args, "use_mp_args_from_checkpoint_args", False):
        if not checkpointing.load_args_from_checkpoint(args):
            raise SystemExit("--use-checkpoint-args: no checkpoint with stored arguments under --load")
    validate_args(args, args_defaults)
    set_args(args)
    from ..utils.log_handler import setup_logging
    setup_logging(getattr(args, "logging_level", None))
    from ..utils.msc import configure_from_args as _configure_msc
    _configure_msc(args)                       # --disable-msc: paths are opened as plain files
    use_cuda = torch.cuda.is_available() and args.distributed_backend == "nccl"
    if use_cuda:
        torch.cuda.set_device(args.local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = dict(backend=args.distributed_backend if use_cuda else "gloo", world_size=args.world_size, rank=args.rank,
                  timeout=timedelta(minutes=args.distributed_timeout_minutes))
        if use_cuda:
            kw["device_id"] = torch.device("cuda", args.local_rank)
        if store is not None:
            kw["store"] = store          # a rendezvous store of the caller's (fresh key space per restart attempt)
        dist.init_process_group(**kw)
    state.initialize_model_parallel(
        tensor_model_parallel_size=args.tensor_model_parallel_size,
        pipeline_model_parallel_size=args.pipeline_model_parallel_size,
        virtual_pipeline_model_parallel_size=args.virtual_pipeline_model_parallel_size,
        context_parallel_size=args.context_parallel_size,
        hierarchical_context_parallel_sizes=getattr(args, "hierarchical_context_parallel_sizes", None),
        expert_model_parallel_size=args.expert_model_parallel_size,
        expert_tensor_parallel_size=args.expert_tensor_parallel_size,
        num_distributed_optimizer_instances=getattr(args, "num_distributed_optimizer_instances", 1),
        nccl_communicator_config_path=getattr(args, "nccl_communicator_config_path", None),
        distributed_timeout_minutes=args.distributed_timeout_minutes,
        order="tp-cp-ep-dp-pp" if not getattr(args, "use_tp_pp_dp_mapping", False) else "tp-cp-ep-pp-dp",
        create_gloo_process_groups=getattr(args, "enable_gloo_process_groups", True),
        high_priority_stream_groups=getattr(args, "high_priority_stream_groups", None) or ())
    seed = args.seed + 100 * state.get_pipeline_model_parallel_rank()
    if getattr(args, "data_parallel_random_init", False):
        seed += 10 * state.get_data_parallel_rank()
    import random
    import numpy as np
    random.seed(seed)
    np.random.seed(seed)
    model_parallel_cuda_manual_seed(seed)
    _TIMERS = Timers(args.timing_log_level, args.timing_log_option)
    if getattr(args, "tensorboard_dir", None) and args.rank == args.world_size - 1:
        try:
            from torch.utils.tensorboard import SummaryWriter
            _WRITER = SummaryWriter(log_dir=args.tensorboard_dir, max_queue=args.tensorboard_queue_size)
        except Exception:
            _WRITER = None
    args.tokenizer = None
    if getattr(args, "tokenizer_type", None):
        args.tokenizer = build_tokenizer(args)
    return args


def cyclic_iter(it):
    while True:
        for x in it:
            yield x


def build_train_valid_test_data_iterators(provider: Callable, args):
    """Only the first tensor-parallel rank reads data; the others receive it by broadcast."""
    from ..data.gpt_dataset import build_pretraining_data_loader
    train_iters = args.train_iters
    eval_iters = (train_iters // args.eval_interval + 1) * args.eval_iters if args.eval_interval else 0
    sizes = [train_iters * args.global_batch_size, eval_iters * args.global_batch_size,
             args.eval_iters * args.global_batch_size]
    train_it = valid_it = test_it = None
    if state.get_tensor_model_parallel_rank() == 0:
        train_ds, valid_ds, test_ds = provider(sizes)
        dp_rank, dp_size = state.get_data_parallel_rank(), state.get_data_parallel_world_size()
        mk = lambda ds, consumed: build_pretraining_data_loader(ds, consumed, args.micro_batch_size, dp_rank, dp_size,
                                                                args.dataloader_type or "single", args.num_workers,
                                                                args.seed)
        tl, vl, sl = mk(train_ds, args.consumed_train_samples), mk(valid_ds, 0), mk(test_ds, 0)
        train_it = iter(tl) if tl is not None else None
        valid_it = cyclic_iter(vl) if vl is not None else None
        test_it = cyclic_iter(sl) if sl is not None else None
    # every rank of a tensor-parallel group must agree on whether a phase runs: the ranks that do not read data
    # learn it from the one that does (reference: training.py:2857 broadcasts do_train / do_valid / do_test)
    flags = torch.tensor([int(train_it is not None), int(valid_it is not None and args.eval_iters > 0),
                          int(test_it is not None and args.eval_iters > 0)], dtype=torch.int64)
    if state.get_tensor_model_parallel_world_size() > 1:
        import torch.distributed as dist
        backend = dist.get_backend(state.get_tensor_model_parallel_group())
        dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
        flags = flags.to(dev)
        dist.broadcast(flags, state.get_tensor_model_parallel_src_rank(), group=state.get_tensor_model_parallel_group())
    args.do_train, args.do_valid, args.do_test = (bool(x) for x in flags.tolist())
    return train_it, valid_it, test_it


def training_log(loss_dict: Dict, total_loss_dict: Dict, lr: float, iteration: int, loss_scale: float, skipped: int,
                 grad_norm, num_zeros, args, elapsed_per_iter: float, config, tokens_per_iter: int):
    for k, v in loss_dict.items():
        total_loss_dict[k] = total_loss_dict.get(k, 0.0) + float(v)
    total_loss_dict["_n"] = total_loss_dict.get("_n", 0) + 1
    total_loss_dict["_skipped"] = total_loss_dict.get("_skipped", 0) + skipped
    if iteration % args.log_interval != 0:
        return
    n = max(total_loss_dict.pop("_n", 1) - total_loss_dict.get("_skipped", 0), 1)
    skipped_tot = total_loss_dict.pop("_skipped", 0)
    fl = flops_from_config(config, args.global_batch_size, args.seq_length, args.padded_vocab_size or 0)
    throughput = fl / (elapsed_per_iter * 1e12 * args.world_size)
    line = (f" iteration {iteration:8d}/{args.train_iters:8d} | consumed samples: {args.consumed_train_samples:12d} |"
            f" elapsed time per iteration (ms): {elapsed_per_iter * 1000.0:.1f} |"
            f" throughput per GPU (TFLOP/s/GPU): {throughput:.1f} |"
            f" tokens/s/GPU: {tokens_per_iter / elapsed_per_iter / args.world_size:.1f} |"
            f" learning rate: {lr:.6E} | global batch size: {args.global_batch_size:5d} |")
    tb_every = max(getattr(args, "tensorboard_log_interval", 1) or 1, 1)
    for k in list(total_loss_dict.keys()):
        line += f" {k}: {total_loss_dict[k] / n:.6E} |"
        if _WRITER is not None and iteration % tb_every == 0:
            _WRITER.add_scalar(k, total_loss_dict[k] / n, iteration)
        total_loss_dict[k] = 0.0
    line += f" loss scale: {loss_scale:.1f} |"
    if grad_norm is not None:
        line += f" grad norm: {float(grad_norm):.3f} |"
    if num_zeros is not None:
        line += f" num zeros: {int(num_zeros)} |"
    line += f" number of skipped iterations: {skipped_tot:3d} |"
    if _WRITER is not None and iteration % tb_every == 0:
        _WRITER.add_scalar("iteration-time", elapsed_per_iter, iteration)
        _WRITER.add_scalar("learning-rate", lr, iteration)
        _WRITER.add_scalar("throughput", throughput, iteration)
        if grad_norm is not None:
            _WRITER.add_scalar("grad-norm", float(grad_norm), iteration)
        if getattr(args, "log_loss_scale_to_tensorboard", False):
            _WRITER.add_scalar("loss-scale", loss_scale, iteration)
        if getattr(args, "log_world_size_to_tensorboard", False):
            _WRITER.add_scalar("world-size", args.world_size, iteration)
        if torch.cuda.is_available():
            _WRITER.add_scalar("mem-allocated-bytes", torch.cuda.memory_allocated(), iteration)
            _WRITER.add_scalar("mem-max-allocated-bytes", torch.cuda.max_memory_allocated(), iteration)
            if getattr(args, "log_memory_to_tensorboard", False):
                st = torch.cuda.memory_stats()
                _WRITER.add_scalar("mem-reserved-bytes", st.get("reserved_bytes.all.current", 0), iteration)
                _WRITER.add_scalar("mem-allocated-count", st.get("allocation.all.current", 0), iteration)
    print_rank_last(line)
    if getattr(args, "log_progress", False) and getattr(args, "save", None):
        append_to_progress_log(args, f"iteration: {iteration:8d}\tthroughput: {throughput:.1f} TFLOP/s/GPU\t"
                                     f"tokens: {args.consumed_train_samples * args.seq_length}")
    if getattr(args, "log_timers_to_tensorboard", False) and _TIMERS is not None:
        # a collective over all ranks: outside the writer-only branch
        _TIMERS.write(["forward-backward", "optimizer", "save-checkpoint"], _WRITER, iteration,
                      normalizer=args.log_interval, reset=False)
    if _TIMERS is not None:
        _TIMERS.log(normalizer=args.log_interval)


def append_to_progress_log(args, text: str, barrier: bool = False) -> None:
    """--log-progress: one line per event (start, log step, checkpoint) in ``<save>/progress.txt`` - job id, time,
    world size, then the event (reference: megatron/training/training.py:439 ``append_to_progress_log``)."""
    if getattr(args, "save", None) is None:
        return
    if barrier and dist.is_initialized():
        dist.barrier()
    if args.rank != 0:
        return
    os.makedirs(args.save, exist_ok=True)
    job = os.environ.get("SLURM_JOB_ID", os.environ.get("JOB_ID", ""))
    with open(os.path.join(args.save, "progress.txt"), "a") as f:
        f.write(f"{time.strftime('%Y-%m-%d %H:%M:%S')}\tJob ID: {job}\t# GPUs: {args.world_size}\t{text}\n")


def ec_protection_group(args):
    """The ranks whose states form the stripes of the erasure-coded in-memory checkpoint.  Members need not hold
    replicas of anything: parity is computed over whatever bytes each rank contributes, so a tensor x pipeline
    parallel job with a single data-parallel replica is protected by striping over the whole job."""
    choice = getattr(args, "ec_group", "auto")
    dp_group = state.get_data_parallel_group(with_context_parallel=True)
    dp = dist.get_world_size(dp_group) if dist.is_initialized() and dp_group is not None else 1
    m = args.ec_parity_shards
    k = args.ec_data_shards
    need = (k + m) if k is not None else (m + 1)
    if choice == "data-parallel" or (choice == "auto" and dp >= max(need, 2)):
        return dp_group
    return dist.group.WORLD if dist.is_initialized() else dp_group


def argparse_namespace_copy(args, **overrides):
    import copy
    ns = copy.copy(args)
    for k, v in overrides.items():
        setattr(ns, k, v)
    return ns


def params_l2_norm(model) -> torch.Tensor:
    """L2 norm of all parameters of the whole (model-parallel) model: tensor-parallel duplicates and tied copies
    are counted once, the squares are summed over the model-parallel group (reference: training/utils.py
    calc_params_l2_norm)."""
    tp_rank = state.get_tensor_model_parallel_rank() if state.model_parallel_is_initialized() else 0
    sq = None
    for chunk in model:
        for p in chunk.parameters():
            if getattr(p, "shared", False) or not (getattr(p, "tensor_model_parallel", False) or tp_rank == 0):
                continue
            v = p.detach().float().pow(2).sum()
            sq = v if sq is None else sq + v
    if sq is None:
        return torch.zeros(())
    if dist.is_initialized() and state.model_parallel_is_initialized() and state.get_group_size("mp") > 1:
        dist.all_reduce(sq, group=state.get_model_parallel_group())
    return sq.sqrt()


def _teardown_attempt():
    """Leave nothing of a failed attempt behind: parallel groups, process-wide globals, microbatch calculator."""
    try:
        state.destroy_model_parallel()
    except Exception:
        pass
    from .global_vars import unset_global_variables
    try:
        if getattr(get_args(), "inprocess_empty_cuda_cache", False) and torch.cuda.is_available():
            torch.cuda.empty_cache()
    except Exception:
        pass
    unset_global_variables()


def _maybe_host_fault(args, iteration: int, attempt: int) -> None:
    """Host-side fault injection for restart tests: ``MLB_INJECT_HOST_FAULT="<rank>:<iteration>"`` makes that rank
    raise once, in the first attempt, after the given iteration.  Nothing on a GPU is touched."""
    spec = os.environ.get("MLB_INJECT_HOST_FAULT")
    if not spec or attempt != 0:
        return
    r, it = (int(x) for x in spec.split(":"))
    if args.rank == r and iteration == it:
        raise RuntimeError(f"injected host fault on rank {r} after iteration {it}")


def _upcycle_from_dense(args, model, optimizer, model_provider, config):
    """--moe-use-upcycling: ``--load`` names a dense checkpoint.  A dense model of the same layout is built and
    loaded, its weights are spread over the experts, and the run starts at iteration 0 from the upcycled model
    (saved at once when ``--save`` is set).  Reference: megatron/training/training.py (moe_use_upcycling branch),
    core/transformer/moe/upcycling_utils.py ``load_and_upcycle_model``."""
    from ..models.upcycling import dense_args_for_upcycling, upcycle_model
    if args.load is None:
        raise SystemExit("--moe-use-upcycling needs --load <dense checkpoint>")
    if len(model) != 1:
        raise NotImplementedError("upcycling with interleaved pipeline stages")
    dargs = dense_args_for_upcycling(args)
    dcfg = core_transformer_config_from_args(dargs)
    saved = get_args()
    set_args(dargs)
    try:
        dense = get_model(lambda **kw: model_provider(config=dcfg, **kw), dcfg, None, wrap_with_ddp=False)
    finally:
        set_args(saved)
    ld = argparse_namespace_copy(dargs, finetune=True, no_load_optim=True, no_load_rng=True)
    checkpointing.load_checkpoint(dense, None, None, ld, load_dir=args.load)
    rep = upcycle_model(checkpointing._unwrap(dense[0]), checkpointing._unwrap(model[0]),
                        granularity=getattr(args, "moe_upcycling_granularity", 1), seed=args.seed)
    n = sum(1 for v in rep.values() if v not in ("copied", "kept", "router init"))
    print_rank_0(f"upcycled the dense checkpoint {args.load}: {n} expert tensors filled from dense MLPs, "
                 f"{sum(1 for v in rep.values() if v == 'copied')} tensors copied")
    if optimizer is not None:
        optimizer.reload_model_params()
    del dense


def pretrain(train_valid_test_datasets_provider: Callable, model_provider: Callable, forward_step_func: Callable,
             extra_args_provider=None, args_defaults=None, argv=None, inprocess_call_wrapper=None):
    """Full program.  ``model_provider(pre_process, post_process, vp_stage=None)`` builds a model chunk;
    ``forward_step_func(data_iterator, model)`` returns ``(output, loss_func)``.  With ``--inprocess-restart`` the
    body runs inside a restart wrapper: a rank-local failure makes every rank abandon the attempt, tear down its
    groups and start again in the same processes, resuming from the latest checkpoint."""
    av = list(sys.argv[1:] if argv is None else argv)
    if inprocess_call_wrapper is None and "--inprocess-restart" in av:
        from types import SimpleNamespace
        from .inprocess_restart import maybe_wrap_for_inprocess_restart
        def opt(flag, cast, default):
            return cast(av[av.index(flag) + 1]) if flag in av and av.index(flag) + 1 < len(av) else default
        ns = SimpleNamespace(inprocess_restart=True, inprocess_max_iterations=opt("--inprocess-max-iterations", int, None),
                             inprocess_barrier_timeout=opt("--inprocess-barrier-timeout", float, 120.0))
        wrapped, _store = maybe_wrap_for_inprocess_restart(
            lambda **kw: pretrain(train_valid_test_datasets_provider, model_provider, forward_step_func,
                                  extra_args_provider, args_defaults, argv, **kw), ns)
        return wrapped()
    attempt = 0
    if inprocess_call_wrapper is not None:
        inprocess_call_wrapper.finalize = _teardown_attempt
        attempt = inprocess_call_wrapper.attempt
        if attempt:
            print(f"[rank {os.environ.get('RANK', 0)}] in-process restart: attempt {attempt}", flush=True)
    pg_store = None
    if inprocess_call_wrapper is not None:
        # each attempt rendezvouses under its own prefix: keys of a torn-down attempt cannot be picked up again
        pg_store = dist.PrefixStore(f"pg_attempt_{attempt}", inprocess_call_wrapper.store)
    args = initialize_megatron(extra_args_provider, args_defaults, argv=argv, store=pg_store)
    timers = get_timers()
    config = core_transformer_config_from_args(args)
    ocfg, dcfg = optimizer_config_from_args(args), ddp_config_from_args(args)
    timers("model-and-optimizer-setup", 0).start(barrier=True)
    model = get_model(lambda **kw: model_provider(config=config, **kw), config, dcfg)
    head_mult = getattr(args, "head_lr_mult", 1.0) or 1.0
    if head_mult != 1.0:
        # --head-lr-mult: the task heads (classification / decoder heads of the vision programs) learn at a multiple
        # of the backbone's rate (reference: pretrain_vision_classify.py scale_lr_cond)
        optimizer = build_optimizer(ocfg, model, scale_lr_cond=lambda name, p: "head" in name or "linear_decoder" in name,
                                    lr_mult=head_mult)
    else:
        optimizer = build_optimizer(ocfg, model)
    scheduler = get_optimizer_param_scheduler(
        optimizer, lr=args.lr, min_lr=args.min_lr, lr_decay_style=args.lr_decay_style, train_iters=args.train_iters,
        global_batch_size=args.global_batch_size, lr_decay_iters=args.lr_decay_iters,
        lr_warmup_iters=args.lr_warmup_iters, lr_warmup_fraction=args.lr_warmup_fraction,
        lr_warmup_init=args.lr_warmup_init, weight_decay=args.weight_decay,
        start_weight_decay=args.start_weight_decay, end_weight_decay=args.end_weight_decay,
        weight_decay_incr_style=args.weight_decay_incr_style, lr_wsd_decay_style=args.lr_wsd_decay_style,
        lr_wsd_decay_iters=args.lr_wsd_decay_iters, lr_decay_samples=getattr(args, "lr_decay_samples", None),
        lr_warmup_samples=getattr(args, "lr_warmup_samples", 0) or 0,
        lr_wsd_decay_samples=getattr(args, "lr_wsd_decay_samples", None))
    install_callbacks(config, model, optimizer)
    if config.tp_comm_overlap and torch.cuda.is_available():
        from ..ops.tp_fused import attach_fused_tp
        attach_fused_tp(model, config, args.seq_length, args.micro_batch_size)
    iteration, flops_so_far = 0, 0.0
    if getattr(args, "moe_use_upcycling", False):
        # --load names the dense checkpoint; the mixture-of-experts run it seeds must start in a fresh --save
        if args.save and os.path.isfile(checkpointing.get_checkpoint_tracker_filename(args.save)):
            raise SystemExit(f"--moe-use-upcycling: {args.save} already holds a checkpoint; resume from it without "
                             "the flag")
        _upcycle_from_dense(args, model, optimizer, model_provider, config)
    elif args.load is not None:
        iteration, flops_so_far = checkpointing.load_checkpoint(model, optimizer, scheduler, args)
        args.consumed_train_samples = iteration * args.global_batch_size
    if getattr(args, "ckpt_convert_format", None):
        # load in whatever format the checkpoint has, write it again in the requested one, stop
        # (reference: training/training.py --ckpt-convert-format / --ckpt-convert-save)
        out_dir = getattr(args, "ckpt_convert_save", None)
        if args.load is None or out_dir is None:
            raise SystemExit("--ckpt-convert-format needs --load and --ckpt-convert-save")
        conv = argparse_namespace_copy(args, ckpt_format=args.ckpt_convert_format, save=os.path.join(out_dir, args.ckpt_convert_format),
                                       async_save=False)
        checkpointing.save_checkpoint(iteration, model, optimizer, scheduler, conv,
                                      num_floating_point_operations_so_far=flops_so_far)
        print_rank_0(f"converted the checkpoint of iteration {iteration} to {args.ckpt_convert_format} in {conv.save}")
        if dist.is_initialized():
            dist.barrier()
        sys.exit(0)
    if iteration == 0 and getattr(args, "pretrained_checkpoint", None):
        # nothing to resume from: start from the weights of a pre-trained checkpoint (no optimizer state, no
        # iteration count), as --finetune does (reference: training/checkpointing.py load of pretrained_checkpoint)
        ft = argparse_namespace_copy(args, finetune=True, no_load_optim=True, no_load_rng=True)
        checkpointing.load_checkpoint(model, optimizer, scheduler, ft, load_dir=args.pretrained_checkpoint)
    timers("model-and-optimizer-setup").stop()
    ec_manager = None
    if getattr(args, "non_persistent_ckpt_type", None) == "local":
        grp = ec_protection_group(args)
        on_gpu = torch.cuda.is_available() and dist.get_backend(grp) == "nccl" and dist.get_world_size(grp) > 1
        if on_gpu and getattr(args, "ec_device", "auto") != "cpu":
            # parity computed by the peer-memory GF(2^8) kernel, parity held in the peers' HBM, host tier on a
            # side stream; the state size fixes the stripe plan
            from ..checkpoint.ec_gpu import GpuECCheckpoint
            tensors = list(optimizer.local_state_tensors())
            for chunk in model:
                for buf in getattr(chunk, "buffers", []) + getattr(chunk, "expert_buffers", []):
                    tensors.append(buf.param_data)
            nbytes = sum(t.numel() * t.element_size() for t in tensors)
            ec_manager = GpuECCheckpoint(grp, nbytes, args.ec_data_shards, args.ec_parity_shards, args.ec_chunk_bytes,
                                         host_tier=getattr(args, "ec_host_tier", True))
        else:
            ec_manager = ECCheckpointManager(grp, args.ec_data_shards, args.ec_parity_shards, args.ec_chunk_bytes)
    timers("train/valid/test-data-iterators-setup", 0).start(barrier=True)
    train_it, valid_it, test_it = build_train_valid_test_data_iterators(train_valid_test_datasets_provider, args)
    timers("train/valid/test-data-iterators-setup").stop()
    if args.load is not None and checkpointing.LAST_LOADED_RNG_STATE is not None:
        # building the data loaders draws from the host generators (worker base seeds); put the checkpoint's
        # generator states back so that a resumed run continues exactly like the uninterrupted one
        checkpointing.set_rng_state(checkpointing.LAST_LOADED_RNG_STATE)
    timers.log(["model-and-optimizer-setup", "train/valid/test-data-iterators-setup"], barrier=True)
    # always present (disabled when --rerun-mode says so): loss functions validate their result through it
    from .resilience import RerunErrorInjector, set_rerun_state_machine
    inj = RerunErrorInjector(getattr(args, "error_injection_rate", 0) or 0,
                             getattr(args, "error_injection_type", None) or "transient_error")
    rerun = RerunStateMachine(mode=getattr(args, "rerun_mode", None) or "disabled", error_injector=inj)
    rerun.rejected_tracker_filename = getattr(args, "result_rejected_tracker_filename", None)
    set_rerun_state_machine(rerun)
    sig = DistributedSignalHandler().__enter__() if getattr(args, "exit_signal_handler", False) else None
    straggler = None
    if getattr(args, "log_straggler", False):
        port = getattr(args, "straggler_ctrlr_port", 65535)
        straggler = StragglerDetector(enabled=not getattr(args, "disable_straggler_on_startup", False),
                                      port=port if port and port != 65535 else None,
                                      minmax_count=getattr(args, "straggler_minmax_count", 1))
    dp = state.get_data_parallel_world_size()
    nmb = args.global_batch_size // (args.micro_batch_size * dp)
    total_loss: Dict = {}
    start_time = time.time()
    for m in model:
        m.train()
    t_last = time.time()
    if rerun.mode.value != "disabled" and train_it is not None:
        from .resilience import RerunDataIterator
        train_it = RerunDataIterator(train_it)            # a replayed step sees the same batches again
    if args.load is not None and checkpointing.LAST_LOADED_RERUN_STATE is not None and rerun.mode.value != "disabled":
        rerun.load_state_dict(checkpointing.LAST_LOADED_RERUN_STATE)
    reported = 0
    its = [train_it] * len(model) if len(model) > 1 else train_it
    if getattr(args, "manual_gc", False):
        import gc
        gc.disable()                     # collections happen at chosen iterations, on every rank at once
        gc.collect()
    energy = None
    if getattr(args, "log_energy", False):
        from ..utils.energy_monitor import EnergyMonitor
        try:
            energy = EnergyMonitor()
            energy.setup()
            energy.resume()
        except Exception as e:           # no NVML on this host
            print_rank_0(f"energy monitor unavailable: {e}")
            energy = None
    heart = None
    if getattr(args, "enable_ft_package", False):
        from .resilience import HeartbeatMonitor
        heart = HeartbeatMonitor(on_timeout=lambda sec, dt: print(
            f"[rank {args.rank}] no heartbeat for {dt:.0f} s in section '{sec}'", flush=True))
        heart.start_section("step")
    if getattr(args, "record_memory_history", False) and torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(max_entries=100000)
    if getattr(args, "skip_train", False):
        iteration = max(iteration, args.train_iters)
    prof = None
    if getattr(args, "profile", False) and getattr(args, "use_pytorch_profiler", False) and \
            args.rank in (args.profile_ranks or [0]):
        # the torch profiler instead of an external one: idle until the start step, one warm-up step, active to
        # the end step; traces land beside the tensorboard logs (reference: training.py:2219-2236)
        start = max(args.profile_step_start - iteration, 0)
        prof = torch.profiler.profile(
            schedule=torch.profiler.schedule(wait=max(start - 1, 0), warmup=1 if start > 0 else 0,
                                             active=max(args.profile_step_end - args.profile_step_start, 1), repeat=1),
            on_trace_ready=torch.profiler.tensorboard_trace_handler(getattr(args, "tensorboard_dir", None) or "profile"),
            record_shapes=True, with_stack=True)
        prof.start()
    from ..utils.common import configure_nvtx_profiling, nvtx_range_pop, nvtx_range_push
    configure_nvtx_profiling(bool(getattr(args, "profile", False)))
    skip_set = set(getattr(args, "iterations_to_skip", None) or [])
    while iteration < args.train_iters:
        checkpointing.maybe_finalize_async_save(blocking=False)
        if (iteration + 1) in skip_set:
            # --iterations-to-skip: the batches of the step are drawn (so the data order of later steps is
            # unchanged) but no forward / backward / update happens (reference: training.py dummy_train_step)
            if train_it is not None:
                for _ in range(nmb):
                    next(train_it)
            iteration += 1
            args.iteration = iteration
            args.consumed_train_samples += args.global_batch_size
            print_rank_0(f" iteration {iteration}: skipped on request")
            continue
        if getattr(args, "profile", False) and iteration == args.profile_step_start and torch.cuda.is_available() \
                and args.rank in (args.profile_ranks or [0]) and prof is None:
            torch.cuda.cudart().cudaProfilerStart()
        nvtx_range_push(f"iteration {iteration + 1}")
        args.curr_iteration = iteration
        if straggler is not None:
            straggler.start()
        loss_dict, skipped, grad_norm, zeros = train_step(
            forward_step_func, its, model, optimizer, scheduler, config, num_microbatches=nmb,
            seq_length=args.seq_length, micro_batch_size=args.micro_batch_size, global_batch_size=args.global_batch_size,
            rerun_state_machine=rerun)
        nvtx_range_pop(f"iteration {iteration + 1}")
        if straggler is not None:
            straggler.stop()
        if not skipped:
            # models that keep a second set of weights in step with the trained one (the momentum teacher of DINO:
            # reference training.py, update_momentum after the optimizer step)
            for chunk in model:
                hook = getattr(checkpointing._unwrap(chunk), "after_optimizer_step", None)
                if hook is not None:
                    hook(iteration)
        for step_no, diag, what in rerun.diagnostics[reported:]:
            print(f" [rank {args.rank}] result validation, iteration {iteration + 1}: {diag.value} ({what})", flush=True)
        reported = len(rerun.diagnostics)
        stop, code = rerun.should_checkpoint_and_exit()
        if stop:
            # the step reproduced a rejected result here: keep the state from before the step, so that a restart
            # (on other hardware) replays it and tells a faulty device from a real divergence
            if args.save:
                checkpointing.save_checkpoint(iteration, model, optimizer, scheduler, args,
                                              num_floating_point_operations_so_far=flops_so_far,
                                              rerun_state=rerun.state_dict())
            checkpointing.maybe_finalize_async_save(blocking=True)
            print_rank_0(f"exiting at iteration {iteration} with code {code} to replay the step from the checkpoint")
            if dist.is_initialized():
                dist.barrier()
            sys.exit(code or 0)
        if rerun.exit_code is not None:
            print_rank_0(f"result validation failed again after the restart: exiting with code {rerun.exit_code}")
            sys.exit(rerun.exit_code)
        if prof is not None:
            prof.step()
        iteration += 1
        args.iteration = iteration
        _maybe_host_fault(args, iteration, attempt)
        if inprocess_call_wrapper is not None:
            inprocess_call_wrapper.step_barrier(iteration)   # a peer failed: abandon this attempt between steps
        args.consumed_train_samples += args.global_batch_size
        flops_so_far += flops_from_config(config, args.global_batch_size, args.seq_length, args.padded_vocab_size or 0)
        if iteration % args.log_interval == 0:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            now = time.time()
            elapsed = (now - t_last) / args.log_interval
            t_last = now
        else:
            elapsed = 0.0
        if getattr(args, "train_sync_interval", None) and iteration % args.train_sync_interval == 0 \
                and torch.cuda.is_available():
            torch.cuda.synchronize()      # keeps the host from running far ahead of the device
        if getattr(args, "empty_unused_memory_level", 0) and torch.cuda.is_available():
            torch.cuda.empty_cache()
        if getattr(args, "log_params_norm", False) and iteration % args.log_interval == 0:
            print_rank_last(f" iteration {iteration}: params norm: {float(params_l2_norm(model)):.4f}")
        lr = optimizer.param_groups[0]["lr"]
        training_log(loss_dict, total_loss, lr, iteration, float(optimizer.get_loss_scale()), skipped, grad_norm, zeros,
                     args, max(elapsed, 1e-9), config, args.global_batch_size * args.seq_length)
        if straggler is not None and iteration % args.log_interval == 0:
            straggler.report(iteration)
        if heart is not None:
            heart.heartbeat()
        if energy is not None and iteration % args.log_interval == 0:
            joules = energy.lap()
            print_rank_last(f" energy since the last report: {joules:.1f} J "
                            f"({joules / max(args.log_interval * args.global_batch_size * args.seq_length, 1):.4f} J/token)")
            if _WRITER is not None:
                _WRITER.add_scalar("energy-joules", joules, iteration)
        if getattr(args, "manual_gc", False) and getattr(args, "manual_gc_interval", 0) and \
                iteration % args.manual_gc_interval == 0:
            import gc
            gc.collect()
        hash_every = getattr(args, "check_weight_hash_across_dp_replicas_interval", None)
        if hash_every and iteration % hash_every == 0:
            from ..utils.common import check_param_hashes_across_dp_replicas
            if not check_param_hashes_across_dp_replicas(model):
                raise RuntimeError(f"data-parallel replicas hold different weights at iteration {iteration}")
        if getattr(args, "profile", False) and iteration == args.profile_step_end and torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStop()
        if args.eval_interval and iteration % args.eval_interval == 0 and args.do_valid:
            res = evaluate(forward_step_func, valid_it, model, config, eval_iters=args.eval_iters, num_microbatches=nmb,
                           seq_length=args.seq_length, micro_batch_size=args.micro_batch_size)
            print_rank_last(f" validation loss at iteration {iteration} | " +
                            " | ".join(f"{k} value: {v:.6E} | {k} PPL: {math.exp(min(20.0, v)):.6E}"
                                       for k, v in res.items()))
            if _WRITER is not None:
                for k, v in res.items():
                    _WRITER.add_scalar(f"{k} validation", v, iteration)
                    if getattr(args, "log_validation_ppl_to_tensorboard", False):
                        _WRITER.add_scalar(f"{k} validation ppl", math.exp(min(20.0, v)), iteration)
            if getattr(args, "manual_gc", False) and getattr(args, "manual_gc_eval", False):
                import gc
                gc.collect()
        if ec_manager is not None and args.non_persistent_save_interval and \
                iteration % args.non_persistent_save_interval == 0:
            st = checkpointing.save_checkpoint(iteration, model, optimizer, scheduler, args, non_persistent=True,
                                               ec_manager=ec_manager)
            if "encode_ms" in st:        # GPU tier: device-timed snapshot and parity kernels
                when = f" (device times of the save at iteration {int(st['of_iteration'])})" if "of_iteration" in st else ""
                print_rank_0(f" in-memory erasure-coded checkpoint at iteration {iteration}: snapshot "
                             f"{st.get('snapshot_ms', 0.0):.2f} ms, encode {st['encode_ms']:.2f} ms{when}, "
                             f"{st.get('total_s', 0.0):.3f} s on the host")
            elif hasattr(ec_manager, "hdl"):
                print_rank_0(f" in-memory erasure-coded checkpoint at iteration {iteration}: parity and host copy "
                             f"running under the next steps, {st.get('total_s', 0.0):.3f} s on the host")
            else:
                print_rank_0(f" in-memory erasure-coded checkpoint at iteration {iteration}: "
                             f"{st.get('encode_GBps', 0.0):.2f} GB/s encode, {st.get('total_s', 0.0):.3f} s")
        exiting = False
        if sig is not None and any(sig.signals_received()):
            exiting = True
        if getattr(args, "exit_interval", None) and iteration % args.exit_interval == 0:
            exiting = True
        if getattr(args, "exit_duration_in_mins", None) and (time.time() - start_time) / 60.0 > args.exit_duration_in_mins:
            exiting = True
        if args.save and ((args.save_interval and iteration % args.save_interval == 0) or exiting):
            timers("save-checkpoint", 0).start(barrier=True)
            checkpointing.save_checkpoint(iteration, model, optimizer, scheduler, args,
                                          num_floating_point_operations_so_far=flops_so_far)
            timers("save-checkpoint").stop(barrier=True)
            timers.log(["save-checkpoint"])
            if getattr(args, "log_progress", False):
                append_to_progress_log(args, f"Saved checkpoint\tIteration: {iteration}\t"
                                             f"Floating-point operations: {flops_so_far:.2e}")
        if exiting:
            print_rank_0(f"exiting program at iteration {iteration}")
            break
    checkpointing.maybe_finalize_async_save(blocking=True)
    if args.save and iteration % max(args.save_interval or 1, 1) != 0 and iteration > 0:
        checkpointing.save_checkpoint(iteration, model, optimizer, scheduler, args,
                                      num_floating_point_operations_so_far=flops_so_far)
    if args.do_test:
        res = evaluate(forward_step_func, test_it, model, config, eval_iters=args.eval_iters, num_microbatches=nmb,
                       seq_length=args.seq_length, micro_batch_size=args.micro_batch_size)
        print_rank_last(" test loss | " + " | ".join(f"{k} value: {v:.6E}" for k, v in res.items()))
    if prof is not None:
        prof.stop()
    if heart is not None:
        heart.end_section()
        if getattr(args, "calc_ft_timeouts", False):
            heart.calculate_and_persist_timeouts()
        heart.shutdown()
    if energy is not None:
        print_rank_last(f" total energy: {energy.get_total():.1f} J")
        energy.shutdown()
    if getattr(args, "record_memory_history", False) and torch.cuda.is_available():
        path = getattr(args, "memory_snapshot_path", None) or "snapshot.pickle"
        torch.cuda.memory._dump_snapshot(f"{path}.rank{args.rank}")
    if _WRITER is not None:
        _WRITER.flush()
    return model, optimizer, scheduler
