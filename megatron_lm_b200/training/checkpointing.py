"""Checkpoint save / load glue.

Directory layout and state captured follow the reference (megatron/training/checkpointing.py:
tracker file ``latest_checkpointed_iteration.txt`` :228, ``iter_{:07d}`` directories, legacy
``mp_rank_{tp:02d}[_{pp:03d}]/model_optim_rng.pt`` :130, ``generate_state_dict`` :729 with args,
``checkpoint_version`` 3.0, iteration, ``model``/``model{i}``, optimizer, scheduler, RNG states,
rerun-state-machine state and the running FLOP count; load prefers the newest of the persistent
and the in-memory checkpoint :991-1002).  Formats:

* ``torch_dist`` - sharded, reshardable (``checkpoint/sharded.py``), optionally written by a
  background worker after a synchronous device-to-host copy (``--async-save``);
* ``torch``      - one file per model-parallel rank;
* non-persistent ``local`` - erasure-coded in-memory checkpoint (``checkpoint/ec_checkpoint.py``),
  the counterpart of the reference's replicated local checkpoint (:520-544, :870-900).
"""
from __future__ import annotations

import os
import random
import threading
import time
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from ..checkpoint import sharded as ds
from ..parallel import state
from ..parallel.random import get_cuda_rng_tracker

TRACKER = "latest_checkpointed_iteration.txt"


def _unwrap(m):
    while hasattr(m, "module"):
        m = m.module
    return m


def get_checkpoint_tracker_filename(d: str) -> str:
    return os.path.join(d, TRACKER)


def get_checkpoint_name(d: str, iteration: int, release: bool = False, tp_rank=None, pp_rank=None, ep_rank=None,
                        return_base_dir: bool = False) -> str:
    base = os.path.join(d, "release" if release else f"iter_{iteration:07d}")
    if return_base_dir:
        return base
    init = state.model_parallel_is_initialized()
    tp_rank = (state.get_tensor_model_parallel_rank() if init else 0) if tp_rank is None else tp_rank
    pp_rank = (state.get_pipeline_model_parallel_rank() if init else 0) if pp_rank is None else pp_rank
    pp = state.get_pipeline_model_parallel_world_size() if init else 1
    ep = state.get_expert_model_parallel_world_size() if init else 1
    ep_rank = (state.get_expert_model_parallel_rank() if init else 0) if ep_rank is None else ep_rank
    name = f"mp_rank_{tp_rank:02d}" + (f"_{pp_rank:03d}" if pp > 1 else "") + (f"_{ep_rank:03d}" if ep > 1 else "")
    return os.path.join(base, name, "model_optim_rng.pt")


def read_metadata(tracker_filename: str):
    with open(tracker_filename) as f:
        s = f.read().strip()
    if s == "release":
        return 0, True
    return int(s), False


def get_rng_state() -> Dict[str, Any]:
    st = {"random_rng_state": random.getstate(), "np_rng_state": np.random.get_state(),
          "torch_rng_state": torch.get_rng_state(),
          "rng_tracker_states": get_cuda_rng_tracker().get_states()}
    if torch.cuda.is_available():
        st["cuda_rng_state"] = torch.cuda.get_rng_state()
    return st


LAST_LOADED_RNG_STATE: Optional[Dict[str, Any]] = None     # what the latest load_checkpoint restored, if anything
LAST_LOADED_RERUN_STATE: Optional[Dict[str, Any]] = None   # state of the result-validation machine in that checkpoint


def set_rng_state(st: Dict[str, Any]) -> None:
    global LAST_LOADED_RNG_STATE
    LAST_LOADED_RNG_STATE = st
    random.setstate(st["random_rng_state"])
    np.random.set_state(st["np_rng_state"])
    torch.set_rng_state(st["torch_rng_state"])
    if torch.cuda.is_available() and "cuda_rng_state" in st:
        torch.cuda.set_rng_state(st["cuda_rng_state"])
    if st.get("rng_tracker_states"):
        get_cuda_rng_tracker().set_states(st["rng_tracker_states"])


# ----------------------------------------------------------------------------- sharded descriptions
def _coords():
    init = state.model_parallel_is_initialized()
    return dict(tp_rank=state.get_tensor_model_parallel_rank() if init else 0,
                tp_size=state.get_tensor_model_parallel_world_size() if init else 1,
                dp_rank=state.get_data_parallel_rank(with_context_parallel=True) if init else 0,
                pp_rank=state.get_pipeline_model_parallel_rank() if init else 0,
                pp_size=state.get_pipeline_model_parallel_world_size() if init else 1)


def _uniform_layer_stack(m) -> bool:
    """Whether every layer of the model has the same parameters (decided from the configuration, so that all
    pipeline stages agree): only then can a parameter be stored as one tensor with a layer axis."""
    cfg = m.config
    if type(m).__name__ == "MambaModel" or getattr(cfg, "heterogeneous_layers_config_encoded_json", None):
        return False
    freq = getattr(cfg, "moe_layer_freq", 1)
    if getattr(cfg, "num_moe_experts", None) and freq not in (None, 1):
        if isinstance(freq, int) or len(set(freq)) > 1:
            return False
    return True


def model_sharded_state_dicts(model: Sequence[torch.nn.Module]) -> List[Dict[str, ds.ShardedTensor]]:
    c = _coords()
    out = []
    for chunk in model:
        m = _unwrap(chunk)
        off = getattr(getattr(m, "decoder", None), "layer_offset", 0)
        out.append(ds.model_sharded_state_dict(m, tp_rank=c["tp_rank"], tp_size=c["tp_size"], dp_rank=c["dp_rank"],
                                               pp_layer_offset=off, num_layers_global=m.config.num_layers,
                                               stack_layers=_uniform_layer_stack(m)))
    return out


def _part_spans(model_sd, name, p):
    """A parameter that the model's description stores in several pieces along its first dimension (gated FC1
    halves, a Mamba mixer's segments): [(description of the piece, first, one-past-last flat index inside the
    parameter)].  Rows are contiguous, so a flat range of the parameter is a flat range of each piece it crosses."""
    if int(getattr(p, "partition_dim", -1)) != 0 or f"{name}.part0" not in model_sd:
        return None
    spans, at, i = [], 0, 0
    while f"{name}.part{i}" in model_sd:
        d = model_sd[f"{name}.part{i}"]
        n = 1
        for e in d.local_shape:
            n *= int(e)
        spans.append((d, at, at + n))
        at, i = at + n, i + 1
    return spans if at == p.numel() else None


def optimizer_sharded_state_dict(optimizer, model: Sequence[torch.nn.Module],
                                 model_sd: List[Dict[str, ds.ShardedTensor]]) -> Dict[str, Any]:
    """Optimizer state in model space: for every parameter piece this rank owns,
    ``optimizer.state.{fp32_param,exp_avg,exp_avg_sq}.<model key>`` with the parameter's global
    placement and the flattened range of the piece (reference: distrib_optimizer.py:1344-1440)."""
    opts = getattr(optimizer, "chained_optimizers", [optimizer])
    name_of = {}
    for ci, chunk in enumerate(model):
        for n, p in _unwrap(chunk).named_parameters():
            name_of[p] = (ci, n)
        # trained parameters that belong to a wrapper, not to the saved model (a distillation projection layer):
        # their optimizer state is kept under the wrapper's name
        m = chunk
        while hasattr(m, "module"):
            for n, p in m.named_parameters():
                name_of.setdefault(p, (ci, "wrapper." + n))
            m = m.module
    c = _coords()
    out: Dict[str, Any] = {"param_state": {}, "common": []}
    for oi, opt in enumerate(opts):
        out["common"].append(dict(step=opt.step_count, param_groups=[dict(g) for g in opt.param_groups],
                                  grad_scaler=None if opt.grad_scaler is None else opt.grad_scaler.state_dict()))
        for st in opt.states:
            sharded_over_dp = st.sharded
            for piece in st.pieces:
                p = piece["param"]
                ci, n = name_of[p]
                lo = piece["param_start"]
                hi = lo + piece["numel"]
                desc = model_sd[ci].get(n)
                if desc is not None:
                    spans = [(desc, 0, p.numel())]
                else:
                    spans = _part_spans(model_sd[ci], n, p)
                if spans is None:         # pieces along an inner dimension: describe in the parameter's own flat space
                    spans = [(ds.ShardedTensor.from_rank_offsets(
                        f"chunk{ci}.{n}.tp{c['tp_rank']}of{c['tp_size']}.pp{c['pp_rank']}", p.detach(),
                        replica_id=(0, 0, c["dp_rank"])), 0, p.numel())]
                for desc, a, b in spans:
                    s_lo, s_hi = max(lo, a), min(hi, b)
                    if s_lo >= s_hi:
                        continue
                    whole = (s_lo == a and s_hi == b)
                    at = piece["local_start"] + (s_lo - lo)
                    for kind, flat in (("fp32_param", st.master), ("exp_avg", st.exp_avg), ("exp_avg_sq", st.exp_avg_sq)):
                        data = flat[at:at + (s_hi - s_lo)]
                        replica = desc.replica_id if not sharded_over_dp else (desc.replica_id[0], desc.replica_id[1], 0)
                        stn = ds.ShardedTensor(f"optimizer.state.{kind}.{desc.key}",
                                               data if not whole else data.view(desc.local_shape),
                                               torch.float32, desc.local_shape, desc.global_shape, desc.global_offset,
                                               desc.axis_fragmentations, replica, desc.prepend_axis_num, False,
                                               None if whole else slice(s_lo - a, s_hi - a))
                        out["param_state"][f"{oi}.{kind}.{ci}.{n}.{s_lo}"] = stn
    return out


def generate_state_dict(args, model, optimizer, opt_param_scheduler, rng_state, iteration: int, sharded: bool,
                        rerun_state=None, num_floating_point_operations_so_far: float = 0.0) -> Dict[str, Any]:
    sd: Dict[str, Any] = {"args": args, "checkpoint_version": 3.0, "iteration": iteration,
                          "num_floating_point_operations_so_far": num_floating_point_operations_so_far}
    model_sd = model_sharded_state_dicts(model) if sharded else None
    for i, chunk in enumerate(model):
        key = "model" if len(model) == 1 else f"model{i}"
        sd[key] = model_sd[i] if sharded else _unwrap(chunk).state_dict()
    if optimizer is not None and not getattr(args, "no_save_optim", False):
        sd["optimizer"] = optimizer_sharded_state_dict(optimizer, model, model_sd) if sharded else optimizer.state_dict()
        if opt_param_scheduler is not None:
            sd["opt_param_scheduler"] = opt_param_scheduler.state_dict()
    if rerun_state is not None:
        # every rank keeps its own first result of the step under replay
        if sharded and dist.is_initialized():
            sd["rerun_state_machine"] = ds.ShardedObject("rerun_state_machine", rerun_state, (dist.get_world_size(),),
                                                         (dist.get_rank(),))
        else:
            sd["rerun_state_machine"] = rerun_state
    if rng_state is not None and not getattr(args, "no_save_rng", False):
        if sharded:
            c = _coords()
            dp = state.get_data_parallel_world_size(with_context_parallel=True) if state.model_parallel_is_initialized() else 1
            sd["rng_state"] = ds.ShardedObject("rng_state", rng_state, (c["pp_size"], c["tp_size"], dp),
                                               (c["pp_rank"], c["tp_rank"], c["dp_rank"]))
        else:
            sd["rng_state"] = rng_state
    return sd


# ----------------------------------------------------------------------------- torch (legacy layout) helpers
def _dp_coords():
    if not state.model_parallel_is_initialized():
        return 0, 1
    return (state.get_data_parallel_rank(with_context_parallel=True),
            state.get_data_parallel_world_size(with_context_parallel=True))


def _optimizer_is_dp_sharded(optimizer) -> bool:
    opts = getattr(optimizer, "chained_optimizers", [optimizer])
    return any(getattr(st, "sharded", False) for o in opts for st in getattr(o, "states", []))


def _distrib_optim_name(model_file: str) -> str:
    return os.path.join(os.path.dirname(model_file), f"distrib_optim_dp{_dp_coords()[0]:03d}.pt")


def _strip_optimizer_tensors(opt_sd):
    if isinstance(opt_sd, list):
        return [_strip_optimizer_tensors(x) for x in opt_sd]
    return {k: v for k, v in opt_sd.items() if k != "state"}


def _writes_model_file() -> bool:
    """One writer per file name: the file is named after (tp, pp, ep) ranks, so with expert parallelism every
    expert-parallel rank of the first expert-data-parallel replica writes (its experts exist nowhere else)."""
    if not state.model_parallel_is_initialized():
        return True
    if state.get_expert_model_parallel_world_size() > 1:
        return state.get_expert_data_parallel_rank() == 0
    return state.get_data_parallel_rank(with_context_parallel=True) == 0


# ----------------------------------------------------------------------------- async worker
class AsyncCallsQueue:
    """Runs checkpoint writes on a background thread; ``maybe_finalize`` is polled from the
    training loop and all ranks agree before the tracker file is updated (reference:
    dist_checkpointing/strategies/async_utils.py:478)."""

    def __init__(self):
        self.pending: List[tuple] = []

    def schedule(self, fn, finalize_fn):
        t = threading.Thread(target=fn, daemon=True)
        t.start()
        self.pending.append((t, finalize_fn))

    def maybe_finalize(self, blocking: bool = False) -> None:
        still = []
        for t, fin in self.pending:
            if blocking:
                t.join()
            done = torch.tensor([0 if t.is_alive() else 1], dtype=torch.int32)
            if dist.is_initialized() and dist.get_world_size() > 1:
                if torch.cuda.is_available() and dist.get_backend() == "nccl":
                    done = done.cuda()
                dist.all_reduce(done, op=dist.ReduceOp.MIN)
            if int(done.item()) == 1:
                fin()
            else:
                still.append((t, fin))
        self.pending = still

    def close(self):
        self.maybe_finalize(blocking=True)


_async_queue = AsyncCallsQueue()


def maybe_finalize_async_save(blocking: bool = False) -> None:
    _async_queue.maybe_finalize(blocking)


# ----------------------------------------------------------------------------- save / load
def _write_tracker(save_dir: str, iteration: int) -> None:
    if not dist.is_initialized() or dist.get_rank() == 0:
        with open(get_checkpoint_tracker_filename(save_dir), "w") as f:
            f.write(str(iteration))


def cleanup_old_checkpoints(save_dir: str, iteration: int, retain_interval: Optional[int]) -> List[int]:
    """--save-retain-interval N: once iteration ``iteration`` is safely written, every older ``iter_*`` directory
    whose iteration is not a multiple of N is deleted (the newest checkpoint always stays).  Rank 0 only; returns the
    iterations removed (reference: megatron/training/checkpointing.py, save_retain_interval clean-up)."""
    if not retain_interval or (dist.is_initialized() and dist.get_rank() != 0) or not os.path.isdir(save_dir):
        return []
    import re as _re
    import shutil
    removed = []
    for name in os.listdir(save_dir):
        m = _re.match(r"^iter_(\d+)$", name)
        if not m:
            continue
        it = int(m.group(1))
        if it < iteration and it % retain_interval != 0:
            shutil.rmtree(os.path.join(save_dir, name), ignore_errors=True)
            removed.append(it)
    return sorted(removed)


# ----------------------------------------------------------------------------- sharded data parallel (FSDP) models
def _is_fsdp_optimizer(optimizer) -> bool:
    from ..parallel.fsdp import ShardedAdam, TorchOptimizerAdapter
    return isinstance(optimizer, (ShardedAdam, TorchOptimizerAdapter))


def _fsdp_rank_file(base: str) -> str:
    rank = dist.get_rank() if dist.is_initialized() else 0
    return os.path.join(base, f"fsdp_rank_{rank:05d}.pt")


def _save_fsdp(iteration, model, optimizer, scheduler, save_dir, rng, flops):
    """Every rank writes the slices it owns (``fsdp_rank_<r>.pt``): with the custom FSDP units the optimizer's fp32
    master shards are the weights; with torch FSDP2 the local parts of the DTensor parameters and of the torch
    optimizer state.  The layout is tied to the world size it was written with."""
    from ..parallel.fsdp import ShardedAdam
    base = get_checkpoint_name(save_dir, iteration, return_base_dir=True)
    os.makedirs(base, exist_ok=True)
    world = dist.get_world_size() if dist.is_initialized() else 1
    sd = {"iteration": iteration, "world_size": world, "rng_state": rng,
          "num_floating_point_operations_so_far": flops,
          "opt_param_scheduler": scheduler.state_dict() if scheduler is not None else None}
    if isinstance(optimizer, ShardedAdam):
        sd["kind"], sd["optimizer"] = "custom_fsdp", optimizer.state_dict()
    else:
        local = lambda t: t.to_local() if hasattr(t, "to_local") else t
        sd["kind"] = "torch_fsdp2"
        sd["model"] = [{n: local(p.detach()).clone() for n, p in m.module.named_parameters()} for m in model]
        osd = optimizer.state_dict()
        sd["optimizer"] = {"param_groups": osd["param_groups"],
                           "state": {k: {kk: (local(vv).clone() if torch.is_tensor(vv) else vv) for kk, vv in v.items()}
                                     for k, v in osd["state"].items()}}
    torch.save(sd, _fsdp_rank_file(base))
    if dist.is_initialized():
        dist.barrier()
    _write_tracker(save_dir, iteration)


def _load_fsdp(model, optimizer, scheduler, base: str, no_optim: bool, no_rng: bool):
    from ..parallel.fsdp import ShardedAdam
    sd = torch.load(_fsdp_rank_file(base), map_location="cpu", weights_only=False)
    world = dist.get_world_size() if dist.is_initialized() else 1
    if sd["world_size"] != world:
        raise RuntimeError(f"this FSDP checkpoint was written by {sd['world_size']} ranks; {world} are loading it")
    if isinstance(optimizer, ShardedAdam):
        optimizer.load_state_dict(sd["optimizer"])       # master shards -> parameter shards -> re-gather
    else:
        with torch.no_grad():
            for m, saved in zip(model, sd["model"]):
                for n, p in m.module.named_parameters():
                    (p.to_local() if hasattr(p, "to_local") else p).copy_(saved[n])
        if not no_optim:
            if not optimizer.state_dict()["state"]:
                optimizer.materialize_state()
            cur = optimizer.state_dict()
            for k, v in sd["optimizer"]["state"].items():
                for kk, vv in v.items():
                    if torch.is_tensor(vv) and k in cur["state"]:
                        tgt = cur["state"][k][kk]
                        (tgt.to_local() if hasattr(tgt, "to_local") else tgt).copy_(vv)
    if scheduler is not None and sd.get("opt_param_scheduler") is not None and not no_optim:
        scheduler.load_state_dict(sd["opt_param_scheduler"])
    if not no_rng and sd.get("rng_state") is not None:
        set_rng_state(sd["rng_state"])
    return int(sd["iteration"]), float(sd.get("num_floating_point_operations_so_far", 0.0))


def save_checkpoint(iteration: int, model, optimizer, opt_param_scheduler, args, *,
                    num_floating_point_operations_so_far: float = 0.0, rerun_state=None,
                    non_persistent: bool = False, ec_manager=None) -> Dict[str, float]:
    t0 = time.time()
    stats: Dict[str, float] = {}
    # with overlapped parameter gathers the buffers hold the other ranks' new weights only once the next forward
    # pass has walked through them: finish every gather before the weights are read
    for chunk in model:
        sync = getattr(chunk, "force_param_sync", None)
        if sync is not None:
            sync()
    if non_persistent and getattr(args, "non_persistent_ckpt_type", None) == "local":
        if ec_manager is None:
            raise RuntimeError("local non-persistent checkpoints need an ECCheckpointManager")
        tensors = list(optimizer.local_state_tensors())
        for chunk in model:
            for buf in getattr(chunk, "buffers", []) + getattr(chunk, "expert_buffers", []):
                tensors.append(buf.param_data)
        if hasattr(ec_manager, "hdl"):
            # GPU tier: the snapshot is taken on the training stream (a device-to-device copy); parity and the host
            # copy run on the manager's side stream under the following steps.  The figures returned are the device
            # times of the previous save (this one's are not known until it has run).
            stats = dict(ec_manager.save(tensors, iteration, overlap=getattr(args, "ec_overlap", True)))
        else:
            stats = ec_manager.save(tensors, iteration)
        stats["total_s"] = time.time() - t0
        return stats
    save_dir = args.non_persistent_global_ckpt_dir if non_persistent else args.save
    fmt = getattr(args, "ckpt_format", "torch_dist")
    rng = get_rng_state()
    if _is_fsdp_optimizer(optimizer):
        _save_fsdp(iteration, model, optimizer, opt_param_scheduler, save_dir, rng,
                   num_floating_point_operations_so_far)
        stats["total_s"] = time.time() - t0
        return stats
    from ..post_training.checkpointing import has_quantizers, save_quantizer_state
    if fmt == "torch_dist" and has_quantizers(model):
        raise NotImplementedError("a model with post-training quantisers is saved with --ckpt-format torch "
                                  "(quantiser ranges and compressed weights are buffers of the per-rank state dict)")
    if fmt == "torch_dist":
        sd = generate_state_dict(args, model, optimizer, opt_param_scheduler, rng, iteration, True, rerun_state,
                                 num_floating_point_operations_so_far)
        out_dir = get_checkpoint_name(save_dir, iteration, return_base_dir=True)
        if getattr(args, "async_save", False):
            # synchronous device-to-host copy, asynchronous file write
            for _, st in ds.extract_sharded(sd)[0]:
                if st.data is not None:
                    st.data = st.data.detach().to("cpu", copy=True)
            world = dist.get_world_size() if dist.is_initialized() else 1
            if world > 1:
                raise NotImplementedError("async save with several ranks needs the collective-free writer; "
                                          "use synchronous save")
            _async_queue.schedule(lambda: ds.save(sd, out_dir), lambda: _write_tracker(save_dir, iteration))
        else:
            ds.save(sd, out_dir)
            _write_tracker(save_dir, iteration)
    elif fmt == "torch":
        sd = generate_state_dict(args, model, optimizer, opt_param_scheduler, rng, iteration, False, rerun_state,
                                 num_floating_point_operations_so_far)
        name = get_checkpoint_name(save_dir, iteration)
        opt_sd = sd.get("optimizer")
        if opt_sd is not None and _optimizer_is_dp_sharded(optimizer):
            # The distributed optimizer holds 1/dp of master weights and moments on every data-parallel rank, so
            # every rank writes its own shard next to the model file (the reference gathers the shards to rank 0
            # into distrib_optim.pt: megatron/training/checkpointing.py:520-560); the model file keeps the step
            # count and the parameter groups only.
            os.makedirs(os.path.dirname(name), exist_ok=True)
            torch.save({"optimizer": opt_sd, "dp_size": _dp_coords()[1]}, _distrib_optim_name(name))
            sd["optimizer"] = _strip_optimizer_tensors(opt_sd)
        if _writes_model_file():
            os.makedirs(os.path.dirname(name), exist_ok=True)
            torch.save(sd, name)
            save_quantizer_state(model, os.path.dirname(name))
        if dist.is_initialized():
            dist.barrier()
        _write_tracker(save_dir, iteration)
    else:
        raise ValueError(f"unknown checkpoint format {fmt}")
    if not non_persistent and not getattr(args, "async_save", False):
        cleanup_old_checkpoints(save_dir, iteration, getattr(args, "save_retain_interval", None))
    stats["total_s"] = time.time() - t0
    return stats


_ARCH_ARGS = ("num_layers", "hidden_size", "ffn_hidden_size", "seq_length", "num_attention_heads", "num_query_groups",
              "group_query_attention", "kv_channels", "max_position_embeddings", "position_embedding_type",
              "rotary_percent", "rotary_base", "add_position_embedding", "swiglu", "squared_relu", "openai_gelu",
              "normalization", "norm_epsilon", "apply_layernorm_1p", "untie_embeddings_and_output_weights",
              "add_bias_linear", "add_qkv_bias", "qk_layernorm", "num_experts", "moe_router_topk", "moe_ffn_hidden_size",
              "moe_layer_freq", "moe_shared_expert_intermediate_size", "moe_grouped_gemm", "multi_latent_attention",
              "hybrid_override_pattern", "hybrid_attention_ratio", "hybrid_mlp_ratio", "mamba_state_dim",
              "mamba_head_dim", "mamba_num_groups", "is_hybrid_model", "padded_vocab_size", "vocab_size",
              "make_vocab_size_divisible_by", "mtp_num_layers", "window_size")
_MP_ARGS = ("tensor_model_parallel_size", "pipeline_model_parallel_size", "virtual_pipeline_model_parallel_size",
            "num_layers_per_virtual_pipeline_stage", "expert_model_parallel_size", "expert_tensor_parallel_size",
            "context_parallel_size", "sequence_parallel")
_TOKENIZER_ARGS = ("tokenizer_type", "tokenizer_model", "vocab_file", "merge_file", "tiktoken_pattern")


def load_args_from_checkpoint(args, load_dir: Optional[str] = None) -> bool:
    """--use-checkpoint-args: take the model's architecture from the arguments stored in the checkpoint, so that a
    run needs ``--load`` only; --use-mp-args-from-checkpoint-args adds the parallel layout,
    --use-tokenizer-model-from-checkpoint-args the tokenizer files.  Returns False when there is no checkpoint.
    Reference: megatron/training/checkpointing.py:1075-1210 ``load_args_from_checkpoint``."""
    load_dir = load_dir or getattr(args, "load", None)
    if load_dir is None:
        return False
    tracker = get_checkpoint_tracker_filename(load_dir)
    if not os.path.isfile(tracker):
        return False
    iteration, release = read_metadata(tracker)
    base = get_checkpoint_name(load_dir, iteration, release, return_base_dir=True)
    if ds.check_is_distributed_checkpoint(base):
        saved = ds.load_common_state_dict(base).get("args")
    else:
        name = get_checkpoint_name(load_dir, iteration, release, tp_rank=0, pp_rank=0)
        if not os.path.isfile(name):
            cands = sorted(d for d in os.listdir(base) if d.startswith("mp_rank_00"))
            if not cands:
                return False
            name = os.path.join(base, cands[0], "model_optim_rng.pt")
        saved = torch.load(name, map_location="cpu", weights_only=False).get("args")
    if saved is None:
        return False
    get = saved.get if isinstance(saved, dict) else (lambda k, d=None: getattr(saved, k, d))
    names = list(_ARCH_ARGS)
    if getattr(args, "use_mp_args_from_checkpoint_args", False):
        names += list(_MP_ARGS)
    if getattr(args, "use_tokenizer_model_from_checkpoint_args", True):
        names += list(_TOKENIZER_ARGS)
    for k in names:
        v = get(k, None)
        if v is not None:
            setattr(args, k, v)
    return True


def load_checkpoint(model, optimizer, opt_param_scheduler, args, *, load_dir: Optional[str] = None,
                    strict: bool = True):
    """Returns (iteration, num_floating_point_operations_so_far).  (0, 0) when nothing to load."""
    load_dir = load_dir or args.load
    if load_dir is None:
        return 0, 0.0
    tracker = get_checkpoint_tracker_filename(load_dir)
    if not os.path.isfile(tracker):
        if getattr(args, "exit_on_missing_checkpoint", False):
            raise SystemExit(f"no checkpoint found in {load_dir}")
        return 0, 0.0
    iteration, release = read_metadata(tracker)
    if getattr(args, "ckpt_step", None) is not None:
        iteration, release = int(args.ckpt_step), False          # --ckpt-step: a named iteration, not the latest
    base = get_checkpoint_name(load_dir, iteration, release, return_base_dir=True)
    if optimizer is not None and _is_fsdp_optimizer(optimizer):
        return _load_fsdp(model, optimizer, opt_param_scheduler, base, getattr(args, "no_load_optim", False),
                          getattr(args, "no_load_rng", False))
    finetune = getattr(args, "finetune", False)
    no_optim = getattr(args, "no_load_optim", False) or finetune or release
    no_rng = getattr(args, "no_load_rng", False) or finetune or release
    if ds.check_is_distributed_checkpoint(base):
        model_sd = model_sharded_state_dicts(model)
        req: Dict[str, Any] = {}
        for i in range(len(model)):
            req["model" if len(model) == 1 else f"model{i}"] = model_sd[i]
        if optimizer is not None and not no_optim:
            req["optimizer"] = optimizer_sharded_state_dict(optimizer, model, model_sd)
        if not no_rng:
            c = _coords()
            dp = state.get_data_parallel_world_size(with_context_parallel=True) if state.model_parallel_is_initialized() else 1
            req["rng_state"] = ds.ShardedObject("rng_state", None, (c["pp_size"], c["tp_size"], dp),
                                                (c["pp_rank"], c["tp_rank"], c["dp_rank"]))
        if dist.is_initialized():
            req["rerun_state_machine"] = ds.ShardedObject("rerun_state_machine", None, (dist.get_world_size(),),
                                                          (dist.get_rank(),))
        # RNG states are per (pp, tp, dp) position: under a different layout there is nothing to restore
        loaded = ds.load(req, base, strict=strict and not getattr(args, "dist_ckpt_strictness", "") == "ignore_all",
                         optional_objects=("rng_state", "rerun_state_machine"))
        for i, chunk in enumerate(model):
            ds.load_model_from_sharded(_unwrap(chunk), loaded["model" if len(model) == 1 else f"model{i}"])
        if optimizer is not None and not no_optim and "optimizer" in loaded:
            opts = getattr(optimizer, "chained_optimizers", [optimizer])
            common = loaded["optimizer"].get("common", [])
            for opt, cm in zip(opts, common):
                opt.step_count = cm["step"]
                for g, s in zip(opt.param_groups, cm["param_groups"]):
                    g.update(s)
                if opt.grad_scaler is not None and cm.get("grad_scaler"):
                    opt.grad_scaler.load_state_dict(cm["grad_scaler"])
            # tensors were copied in place into the optimizer's flat state by ``load``
            if opt_param_scheduler is not None and "opt_param_scheduler" in loaded:
                opt_param_scheduler.load_state_dict(loaded["opt_param_scheduler"])
        elif optimizer is not None:
            optimizer.reload_model_params()
        if not no_rng and loaded.get("rng_state") is not None:
            try:
                set_rng_state(loaded["rng_state"])
            except Exception:
                pass
        sd = loaded
    else:
        name = get_checkpoint_name(load_dir, iteration, release)
        sd = torch.load(name, map_location="cpu", weights_only=False)
        from ..post_training.checkpointing import maybe_restore_quantizer_state
        maybe_restore_quantizer_state(model, os.path.dirname(name))
        for i, chunk in enumerate(model):
            _unwrap(chunk).load_state_dict(sd["model" if len(model) == 1 else f"model{i}"], strict=strict)
        if optimizer is not None and not no_optim and "optimizer" in sd:
            opt_sd = sd["optimizer"]
            if _optimizer_is_dp_sharded(optimizer):
                shard_file = _distrib_optim_name(name)
                if not os.path.isfile(shard_file):
                    raise FileNotFoundError(
                        f"{shard_file}: the distributed optimizer's shard of this data-parallel rank is missing "
                        "(the torch format cannot change the data-parallel size; use --ckpt-format torch_dist)")
                shard = torch.load(shard_file, map_location="cpu", weights_only=False)
                if shard.get("dp_size") != _dp_coords()[1]:
                    raise RuntimeError("torch-format optimizer shards were written with data-parallel size "
                                       f"{shard.get('dp_size')}, this run has {_dp_coords()[1]}; use torch_dist")
                opt_sd = shard["optimizer"]
            optimizer.load_state_dict(opt_sd)
            if opt_param_scheduler is not None and "opt_param_scheduler" in sd:
                opt_param_scheduler.load_state_dict(sd["opt_param_scheduler"])
        elif optimizer is not None:
            optimizer.reload_model_params()
        if not no_rng and "rng_state" in sd:
            set_rng_state(sd["rng_state"])
    if finetune or release:
        return 0, 0.0
    global LAST_LOADED_RERUN_STATE
    LAST_LOADED_RERUN_STATE = sd.get("rerun_state_machine")
    return int(sd.get("iteration", iteration)), float(sd.get("num_floating_point_operations_so_far", 0.0))
