"""Command-line arguments: parse -> validate -> config dataclasses.

Three stages as in the reference (megatron/training/arguments.py: ``parse_args``,
``validate_args`` :329-1078, ``core_transformer_config_from_args`` :1100-1170): the parser is
generated from ``flag_table.FLAGS``; ``validate_args`` derives the data-parallel size, virtual
pipeline size, ``params_dtype``, padded vocabulary and microbatch count and enforces the
combination rules; converters copy same-named fields into ``TransformerConfig``,
``OptimizerConfig`` and ``DistributedDataParallelConfig``.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
from typing import Callable, List, Optional

import torch

from ..config import (DistributedDataParallelConfig, MLATransformerConfig, OptimizerConfig, TransformerConfig)
from .flag_table import FLAGS


def _moe_freq(x: str):
    """int, or a python-style list expression such as "([0]*3+[1]*1)*3"."""
    try:
        return int(x)
    except ValueError:
        allowed = set("0123456789[],()*+ ")
        if not set(x) <= allowed:
            raise argparse.ArgumentTypeError(f"bad --moe-layer-freq {x!r}")
        return list(eval(x, {"__builtins__": {}}, {}))


_TYPES = {"int": int, "float": float, "str": str, "bool": bool, "moe_freq": _moe_freq}
_SPECIAL_DEFAULTS = {"--initial-loss-scale": 2 ** 32, "--local-rank": int(os.getenv("LOCAL_RANK", "0")),
                     "--inprocess-active-world-size": int(os.getenv("WORLD_SIZE", "1"))}
_SPECIAL_CHOICES = {"--timing-log-level": [0, 1, 2],
                    "--dist-ckpt-strictness": ["assume_ok_unexpected", "log_unexpected", "log_all", "raise_unexpected",
                                               "raise_all", "return_unexpected", "return_all", "ignore_all"]}


def build_parser(extra_args_provider: Optional[Callable] = None) -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="megatron_lm_b200 arguments", allow_abbrev=False)
    groups = {}
    seen = set()
    for group, flags, kw in FLAGS:
        if flags[0] in seen:
            continue
        seen.add(flags[0])
        g = groups.setdefault(group, parser.add_argument_group(title=group))
        kw = dict(kw)
        if isinstance(kw.get("type"), str) and kw["type"].startswith("@"):
            kw["type"] = _TYPES.get(kw["type"][1:], str)
        elif "type" in kw and kw["type"] is None:
            kw.pop("type")
        if flags[0] in _SPECIAL_DEFAULTS:
            kw["default"] = _SPECIAL_DEFAULTS[flags[0]]
        if flags[0] in _SPECIAL_CHOICES:
            kw["choices"] = _SPECIAL_CHOICES[flags[0]]
        elif "choices" in kw and kw["choices"] is None:
            kw.pop("choices")
        if kw.get("default") == "float32":
            kw["default"] = torch.float32
        if kw.get("action") in ("store_true", "store_false"):
            kw.pop("type", None)
            kw.pop("choices", None)
        g.add_argument(*flags, **kw)
    # flags of this framework that the reference does not have
    g = parser.add_argument_group(title="erasure-coded in-memory checkpoint")
    g.add_argument("--ec-data-shards", type=int, default=None, help="k: data members per stripe (default group size - m)")
    g.add_argument("--ec-parity-shards", type=int, default=1, help="m: parity members per stripe (losses tolerated)")
    g.add_argument("--ec-chunk-bytes", type=int, default=1 << 20)
    g.add_argument("--ec-group", default="auto", choices=["auto", "data-parallel", "world"],
                   help="ranks that protect one another: the data-parallel group (replicas of one model shard), or "
                        "every rank of the job - each rank's state is a stripe member whatever it holds, so tensor- and "
                        "pipeline-parallel layouts without data parallelism are protected too.  auto: the data-parallel "
                        "group when it has at least k + m ranks, else the world")
    g.add_argument("--no-ec-overlap", dest="ec_overlap", action="store_false",
                   help="GPU tier: wait for the parity kernel and the host copy instead of running them under the next steps")
    g.add_argument("--no-ec-host-tier", dest="ec_host_tier", action="store_false",
                   help="GPU tier: keep snapshot and parity in the GPUs' memory only (no pinned-host copy)")
    g.add_argument("--ec-device", default="auto", choices=["auto", "gpu", "cpu"],
                   help="where parity is computed and held: peer GPUs' memory (auto on NCCL jobs) or host memory")
    g = parser.add_argument_group(title="peer-memory kernels")
    g.add_argument("--peer-memory-collectives", action="store_true",
                   help="(default) distributed optimizer: gradient reduce-scatter as a pull kernel over NVLink peer memory, "
                        "overlapped with backward, and AdamW storing new weights into every rank's parameter buffer "
                        "(data-parallel group of at most eight GPUs inside one node; NCCL elsewhere)")
    g.add_argument("--no-peer-memory-collectives", action="store_true",
                   help="distributed optimizer through NCCL reduce-scatter / all-gather only")
    g.add_argument("--cross-entropy-peer-exchange", action="store_true",
                   help="vocab-parallel cross entropy exchanges its row statistics through peer memory instead of all-reduces")
    if extra_args_provider is not None:
        parser = extra_args_provider(parser)
    return parser


def parse_args(extra_args_provider: Optional[Callable] = None, ignore_unknown_args: bool = False, argv=None):
    parser = build_parser(extra_args_provider)
    if ignore_unknown_args:
        args, _ = parser.parse_known_args(argv)
    else:
        args = parser.parse_args(argv)
    args.rank = int(os.getenv("RANK", "0"))
    args.world_size = int(os.getenv("WORLD_SIZE", "1"))
    return args


def validate_args(args, defaults: Optional[dict] = None):
    """Derive dependent values and reject inconsistent combinations."""
    for k, v in (defaults or {}).items():
        if getattr(args, k, None) is None:
            setattr(args, k, v)
    tp, pp, cp = args.tensor_model_parallel_size, args.pipeline_model_parallel_size, args.context_parallel_size
    model_size = tp * pp * cp
    if args.world_size % model_size != 0:
        raise ValueError(f"world size ({args.world_size}) is not divisible by tp ({tp}) x pp ({pp}) x cp ({cp})")
    args.data_parallel_size = args.world_size // model_size
    if args.expert_tensor_parallel_size is None:
        args.expert_tensor_parallel_size = tp
    # batch sizes
    if args.micro_batch_size is None or args.micro_batch_size <= 0:
        raise ValueError("--micro-batch-size must be set")
    if args.global_batch_size is None:
        args.global_batch_size = args.micro_batch_size * args.data_parallel_size
    if args.global_batch_size % (args.micro_batch_size * args.data_parallel_size) != 0:
        raise ValueError("global batch size must be a multiple of micro batch size x data parallel size")
    # virtual pipeline
    if args.num_layers_per_virtual_pipeline_stage is not None:
        if pp <= 1:
            raise ValueError("interleaved schedule needs pipeline parallelism")
        if args.num_layers % (pp * args.num_layers_per_virtual_pipeline_stage) != 0:
            raise ValueError("layers per pipeline stage must be divisible by layers per virtual stage")
        args.virtual_pipeline_model_parallel_size = (args.num_layers // pp) // args.num_layers_per_virtual_pipeline_stage
    elif getattr(args, "num_virtual_stages_per_pipeline_rank", None) is not None:
        args.virtual_pipeline_model_parallel_size = args.num_virtual_stages_per_pipeline_rank
    else:
        args.virtual_pipeline_model_parallel_size = None
    if args.virtual_pipeline_model_parallel_size == 1:
        args.virtual_pipeline_model_parallel_size = None
    if args.overlap_p2p_comm is None if hasattr(args, "overlap_p2p_comm") else False:
        args.overlap_p2p_comm = False
    # precision
    if args.fp16 and args.bf16:
        raise ValueError("--fp16 and --bf16 are mutually exclusive")
    args.params_dtype = torch.float16 if args.fp16 else torch.bfloat16 if args.bf16 else torch.float32
    if args.bf16 and not args.accumulate_allreduce_grads_in_fp32:
        args.accumulate_allreduce_grads_in_fp32 = True
    # parallel feature combinations
    if args.sequence_parallel and tp == 1:
        args.sequence_parallel = False
    if cp > 1 and args.seq_length % (2 * cp) != 0:
        raise ValueError("seq-length must be divisible by 2 x context-parallel-size")
    if args.overlap_param_gather and not (args.use_distributed_optimizer and args.overlap_grad_reduce):
        raise ValueError("--overlap-param-gather needs --use-distributed-optimizer and --overlap-grad-reduce")
    if args.tp_comm_overlap and not args.sequence_parallel:
        raise ValueError("--tp-comm-overlap needs --sequence-parallel")
    if getattr(args, "replication", False) and getattr(args, "non_persistent_ckpt_type", None) != "local":
        raise ValueError("--replication needs --non-persistent-ckpt-type local")
    if getattr(args, "replication", False):
        # the reference's clique replication (a copy on factor - 1 other ranks) is the code with one data member and
        # factor - 1 parity members per stripe: every parity member then IS a copy.  The erasure-coded manager
        # places the members itself, so --replication-jump (the rank distance between copies) has nothing to set.
        factor = getattr(args, "replication_factor", 2) or 2
        if factor < 2:
            raise ValueError("--replication-factor must be at least 2")
        args.ec_data_shards, args.ec_parity_shards = 1, factor - 1
    # model sizes
    if args.num_layers is None and (getattr(args, "decoder_num_layers", None) or getattr(args, "encoder_num_layers", None)):
        args.num_layers = getattr(args, "decoder_num_layers", None) or args.encoder_num_layers
    for req in ("num_layers", "hidden_size", "num_attention_heads"):
        if getattr(args, req) is None:
            raise ValueError(f"--{req.replace('_', '-')} is required")
    if args.ffn_hidden_size is None:
        args.ffn_hidden_size = int((4 * args.hidden_size * 2 / 3) / 64) * 64 if args.swiglu else 4 * args.hidden_size
    if args.kv_channels is None:
        args.kv_channels = args.hidden_size // args.num_attention_heads
    if not args.group_query_attention:
        args.num_query_groups = args.num_attention_heads
    if args.seq_length is None:
        raise ValueError("--seq-length is required")
    if args.max_position_embeddings is None:
        args.max_position_embeddings = args.seq_length
    if args.position_embedding_type == "learned_absolute" and args.max_position_embeddings < args.seq_length:
        raise ValueError("max-position-embeddings must cover seq-length")
    if args.lr is not None and args.min_lr is not None and args.min_lr > args.lr:
        raise ValueError("--min-lr exceeds --lr")
    if args.save is not None and args.save_interval is None:
        raise ValueError("--save needs --save-interval")
    # --data-args-path: a text file with what --data-path would hold; --per-split-data-args-path: a JSON file with
    # "train" / "valid" / "test" lists (reference: training/arguments.py data group, utils.get_blend_and_blend_per_split)
    if getattr(args, "data_args_path", None):
        with open(args.data_args_path) as f:
            args.data_path = f.read().split()
    if getattr(args, "per_split_data_args_path", None):
        import json as _json
        with open(args.per_split_data_args_path) as f:
            per = _json.load(f)
        for split in ("train", "valid", "test"):
            if per.get(split):
                setattr(args, f"{split}_data_path", [str(x) for x in per[split]])
    # one corpus (or mock data) without an explicit split: the customary 969 / 30 / 1 parts
    if getattr(args, "split", None) is None and (getattr(args, "mock_data", False) or getattr(args, "data_path", None)) \
            and not getattr(args, "train_data_path", None):
        args.split = "969,30,1"
    # iteration-based vs sample-based
    if args.train_iters is not None and args.train_samples is not None:
        raise ValueError("give either --train-iters or --train-samples")
    if args.train_samples is not None:
        args.train_iters = args.train_samples // args.global_batch_size
    if args.lr_warmup_fraction is not None and args.lr_warmup_iters not in (0, None):
        raise ValueError("give either --lr-warmup-fraction or --lr-warmup-iters")
    # recompute
    if args.recompute_activations:
        args.recompute_granularity = "selective"
    if args.recompute_granularity == "selective" and args.recompute_method is not None:
        raise ValueError("recompute method does not apply to selective recompute")
    if args.distribute_saved_activations and args.sequence_parallel:
        raise ValueError("--distribute-saved-activations is incompatible with --sequence-parallel")
    # MoE
    if args.num_experts is not None:
        if args.num_experts % args.expert_model_parallel_size != 0:
            raise ValueError("num-experts must be divisible by expert-model-parallel-size")
        if args.moe_ffn_hidden_size is None:
            args.moe_ffn_hidden_size = args.ffn_hidden_size
    elif args.expert_model_parallel_size > 1:
        raise ValueError("expert parallelism needs --num-experts")
    # deterministic mode
    if getattr(args, "deterministic_mode", False):
        algo = os.getenv("NCCL_ALGO", "")
        if args.world_size > 1 and not any(a in algo for a in ("Tree", "Ring", "CollnetDirect", "CollnetChain", "^NVLS")):
            raise ValueError("deterministic mode needs NCCL_ALGO set to a deterministic algorithm")
        torch.use_deterministic_algorithms(True, warn_only=True)
    # aliases and derived values of flags that only rename or refine another setting
    if getattr(args, "use_rotary_position_embeddings", False):
        args.position_embedding_type = "rope"
    if getattr(args, "grad_reduce_in_bf16", False):
        args.accumulate_allreduce_grads_in_fp32 = False
    for flag, field in (("decoder_first_pipeline_num_layers", "num_layers_in_first_pipeline_stage"),
                        ("decoder_last_pipeline_num_layers", "num_layers_in_last_pipeline_stage")):
        v = getattr(args, flag, None)
        if v is not None:
            if pp <= 1:
                raise ValueError(f"--{flag.replace('_', '-')} needs pipeline parallelism")
            setattr(args, field, v)
    # sample-based learning-rate schedule
    if getattr(args, "lr_decay_samples", None) is not None and args.lr_decay_iters is not None:
        raise ValueError("give either --lr-decay-iters or --lr-decay-samples")
    if getattr(args, "lr_warmup_samples", 0) and args.lr_warmup_iters not in (0, None):
        raise ValueError("give either --lr-warmup-iters or --lr-warmup-samples")
    check_unused_flags(args)
    args.padded_vocab_size = getattr(args, "padded_vocab_size", None)
    args.consumed_train_samples = 0
    args.consumed_valid_samples = 0
    args.iteration = 0
    return args


# Flags of the reference's command line that this framework parses (so launch scripts carry over) but does not act
# on.  "warn": setting it changes nothing that affects results; a warning says so.  "refuse": it would change
# numerics, the parallel layout or what a checkpoint contains, so a run that asks for it stops instead of silently
# training something else.  Every flag of the table in flag_table.py that no module reads must be listed here
# (tests/test_arguments_and_utils.py enumerates them).
_W, _R = "warn", "refuse"
UNUSED_FLAGS = {
    # kernel / implementation selectors whose one implementation here is always on
    "transformer_impl": (_W, "one implementation: the native sm_100a kernels"),
    "te_rng_tracker": (_W, "the native RNG tracker is always used"),
    "use_flash_attn": (_W, "flash attention is the only attention kernel"),
    "no_persist_layer_norm": (_W, "one norm kernel"),
    "bias_swiglu_fusion": (_W, "SwiGLU is always a fused kernel"),
    "deprecated_use_mcore_models": (_W, "deprecated in the reference"),
    "use_legacy_models": (_R, "the legacy model classes are not built"),
    "checkpoint_activations": (_R, "deprecated: use --recompute-granularity full --recompute-method uniform"),
    "onnx_safe": (_W, "no ONNX export path"),
    "nccl_all_reduce_for_prefill": (_W, "inference prefill uses the same collectives as training"),
    "scatter_gather_tensors_in_pipeline": (_W, "pipeline transfers always carry the sequence-parallel shard"),
    "lazy_mpu_init": (_R, "external model-parallel initialisation is not supported"),
    "model_parallel_size": (_R, "old name of --tensor-model-parallel-size"),
    "align_grad_reduce": (_W, "gradient reductions of pipeline stages are launched per chunk as they complete"),
    "tp_comm_overlap_cfg": (_W, "the fused tensor-parallel kernels take no user-buffer configuration"),
    "enable_experimental": (_W, "no experimental-API gate"),
    "disable_mamba_mem_eff_path": (_W, "one Mamba forward path"),
    "kitchen_config_file": (_R, "the Kitchen quantisation back end is not built"),
    "kitchen_recipe_number": (_R, "the Kitchen quantisation back end is not built"),
    # inference engine knobs read by the engines' own constructors, not from the training arguments
    "inference_batch_times_seqlen_threshold": (_W, "inference uses no pipelined micro-batching threshold"),
    "inference_dynamic_batching_num_cuda_graphs": (_W, "the dynamic engine captures no graphs"),
    # Retro / biencoder / vision programs that are not (fully) built
    "retro_add_retriever": (_W, "pretrain_retro.py always builds the retriever"),
    "retro_cyclic_train_iters": (_R, "cyclic Retro training is not built"),
    "block_data_path": (_R, "block-data files of the REALM index are not read: the evidence index is built from --evidence-data-path into --embedding-path"),
    "data_sharding": (_W, "the sampler always gives each data-parallel rank its own part"),
    "vision_pretraining_type": (_W, "the program that is launched (pretrain_vision_classify / _dino / _inpaint) is the choice"),
    "vision_pretraining": (_W, "the program that is launched (pretrain_vision_classify / _dino / _inpaint) is the choice; the flag selects nothing"),
    # resilience / logging services that run with fixed settings here
    "run_workload_inspector_server": (_W, "no workload-inspector server"),
    "inprocess_monitor_thread_interval": (_W, "the restart wrapper polls once per step"),
    "inprocess_monitor_process_interval": (_W, "the restart wrapper polls once per step"),
    "inprocess_progress_watchdog_interval": (_W, "the restart wrapper polls once per step"),
    "inprocess_heartbeat_interval": (_W, "the restart wrapper polls once per step"),
    "inprocess_soft_timeout": (_W, "one timeout: --inprocess-barrier-timeout"),
    "inprocess_hard_timeout": (_W, "one timeout: --inprocess-barrier-timeout"),
    "inprocess_heartbeat_timeout": (_W, "one timeout: --inprocess-barrier-timeout"),
    "inprocess_completion_timeout": (_W, "one timeout: --inprocess-barrier-timeout"),
    "inprocess_last_call_wait": (_W, "no last-call phase"), "inprocess_termination_grace_time": (_W, "no external monitor process"),
    "inprocess_granularity": (_W, "restarts are per rank"), "inprocess_active_world_size": (_R, "spare ranks are not built"),
    "log_throughput": (_W, "throughput is part of every log line"),
    "adlr_autoresume_interval": (_W, "no cluster auto-resume service"),
    # checkpoint options
    "load_main_params_from_ckpt": (_R, "loading fp32 main parameters separately is not built"),
    "non_persistent_local_ckpt_dir": (_W, "local checkpoints live in memory (erasure-coded), not in a directory"),
    "non_persistent_local_ckpt_algo": (_W, "the in-memory checkpoint has one algorithm (erasure coding)"),
    "use_dist_ckpt_deprecated": (_W, "deprecated in the reference"), "dist_ckpt_format_deprecated": (_W, "deprecated in the reference"),
    "use_persistent_ckpt_worker": (_W, "asynchronous saves use one background thread"),
    "auto_detect_ckpt_format": (_W, "the format of a checkpoint is always detected at load"),
    "ckpt_convert_update_legacy_dist_opt_format": (_R, "the legacy distributed-optimizer format is not read"),
    "ckpt_fully_parallel_save_deprecated": (_W, "sharded saves are always spread over the data-parallel ranks"),
    "ckpt_fully_parallel_save": (_W, "sharded saves are always spread over the data-parallel ranks"),
    "ckpt_fully_parallel_load": (_W, "sharded loads read each piece once per data-parallel group"),
    "ckpt_assume_constant_structure": (_W, "no save-plan cache"),
    "load_model_opt_format": (_R, "ModelOpt checkpoints are not read"),
    "replication_jump": (_W, "the in-memory checkpoint manager chooses where the copies of a stripe live"),
}


def check_unused_flags(args, defaults: Optional[dict] = None) -> List[str]:
    """Warn about (or refuse) every flag that was given a non-default value but that nothing here acts on.
    Returns the warnings (also sent to ``warnings.warn``)."""
    import warnings
    if defaults is None:
        defaults = _parser_defaults()
    out = []
    for dest, (kind, why) in UNUSED_FLAGS.items():
        if not hasattr(args, dest):
            continue
        v = getattr(args, dest)
        if v == defaults.get(dest) or (v in (None, False, [], 0) and defaults.get(dest) in (None, False, [], 0)):
            continue
        flag = "--" + dest.replace("_", "-")
        if kind == _R:
            raise ValueError(f"{flag} (= {v!r}) is not supported: {why}")
        msg = f"{flag} (= {v!r}) has no effect here: {why}"
        warnings.warn(msg)
        out.append(msg)
    return out


_DEFAULTS_CACHE: Optional[dict] = None


def _parser_defaults() -> dict:
    global _DEFAULTS_CACHE
    if _DEFAULTS_CACHE is None:
        p = build_parser()
        _DEFAULTS_CACHE = {a.dest: a.default for a in p._actions}
    return _DEFAULTS_CACHE


def _copy_fields(cls, args, overrides=None):
    kw = {}
    for f in dataclasses.fields(cls):
        if hasattr(args, f.name) and f.init:
            v = getattr(args, f.name)
            if v is not None or f.default is None:
                kw[f.name] = v
    kw.update(overrides or {})
    return kw


def core_transformer_config_from_args(args, config_class=None) -> TransformerConfig:
    cls = config_class or (MLATransformerConfig if getattr(args, "multi_latent_attention", False) else TransformerConfig)
    ov = dict(
        params_dtype=args.params_dtype, pipeline_dtype=args.params_dtype, deallocate_pipeline_outputs=True,
        batch_p2p_comm=not getattr(args, "overlap_p2p_comm", False), num_moe_experts=args.num_experts,
        rotary_interleaved=getattr(args, "rotary_interleaved", False),
        layernorm_epsilon=getattr(args, "norm_epsilon", 1e-5),
        layernorm_zero_centered_gamma=getattr(args, "apply_layernorm_1p", False),
        gated_linear_unit=bool(args.swiglu), activation_func="silu" if args.swiglu else
        ("squared_relu" if getattr(args, "squared_relu", False) else
         ("openai_gelu" if getattr(args, "openai_gelu", False) else "gelu")),
        add_bias_linear=getattr(args, "add_bias_linear", True),
        bias_activation_fusion=getattr(args, "bias_gelu_fusion", True), position_embedding_type=args.position_embedding_type,
        rotary_percent=getattr(args, "rotary_percent", 1.0), rotary_base=getattr(args, "rotary_base", 10000),
        max_position_embeddings=args.max_position_embeddings,
        share_embeddings_and_output_weights=not getattr(args, "untie_embeddings_and_output_weights", False),
        num_query_groups=args.num_query_groups if args.group_query_attention else None,
        cp_comm_type=(args.cp_comm_type[0] if isinstance(getattr(args, "cp_comm_type", None), list)
                      and len(args.cp_comm_type) == 1 else getattr(args, "cp_comm_type", None)),
    )
    kw = _copy_fields(cls, args, ov)
    if getattr(args, "heterogeneous_layers_config_path", None) and not kw.get("heterogeneous_layers_config_encoded_json"):
        with open(args.heterogeneous_layers_config_path) as f:
            kw["heterogeneous_layers_config_encoded_json"] = f.read()
    for k in ("init_method", "output_layer_init_method", "embedding_init_method", "timers", "finalize_model_grads_func",
              "grad_scale_func", "no_sync_func", "grad_sync_func", "param_sync_func", "_cpu_offloading_context"):
        kw.pop(k, None)
    if getattr(args, "init_method_xavier_uniform", False):
        kw["init_method"] = torch.nn.init.xavier_uniform_
    return cls(**kw)


def optimizer_config_from_args(args) -> OptimizerConfig:
    kw = _copy_fields(OptimizerConfig, args)
    kw.pop("timers", None)
    kw["params_dtype"] = args.params_dtype
    for name in ("main_grads_dtype", "main_params_dtype", "exp_avg_dtype", "exp_avg_sq_dtype"):
        v = kw.get(name)
        if isinstance(v, str):
            kw[name] = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}.get(v, torch.float32)
    return OptimizerConfig(**kw)


def ddp_config_from_args(args) -> DistributedDataParallelConfig:
    kw = _copy_fields(DistributedDataParallelConfig, args)
    kw["grad_reduce_in_fp32"] = args.accumulate_allreduce_grads_in_fp32
    kw["check_for_nan_in_grad"] = getattr(args, "check_for_nan_in_loss_and_grad", False)
    kw["bucket_size"] = getattr(args, "ddp_bucket_size", None)
    kw["average_in_collective"] = getattr(args, "ddp_average_in_collective", False)
    kw["pad_buckets_for_high_nccl_busbw"] = getattr(args, "ddp_pad_buckets_for_high_nccl_busbw", False)
    kw["peer_memory_collectives"] = not getattr(args, "no_peer_memory_collectives", False)
    kw["num_buckets"] = getattr(args, "ddp_num_buckets", None)
    if getattr(args, "cross_entropy_peer_exchange", False):
        import os
        os.environ["MLB_CE_PEER"] = "1"
    return DistributedDataParallelConfig(**kw)


def load_yaml_args(path: str, args):
    """``--yaml-cfg``: overlay a YAML mapping (flat or nested by section) onto parsed arguments
    (reference: megatron/training/yaml_arguments.py:442)."""
    import yaml
    with open(path) as f:
        cfg = yaml.safe_load(f)

    def flat(d):
        for k, v in d.items():
            if isinstance(v, dict):
                yield from flat(v)
            else:
                yield k, v
    for k, v in flat(cfg):
        setattr(args, k, v)
    return args


_GLOBAL_ARGS = None


def set_args(args):
    global _GLOBAL_ARGS
    _GLOBAL_ARGS = args


def get_args():
    if _GLOBAL_ARGS is None:
        raise RuntimeError("arguments are not initialised")
    return _GLOBAL_ARGS


def validate_yaml(args, defaults=None):
    """Validation of a YAML-built namespace: the same rules as the command line
    (reference: megatron/training/yaml_arguments.py:41)."""
    return validate_args(args, defaults)


def core_transformer_config_from_yaml(args, transfomer_key: str = "language_model"):
    """``TransformerConfig`` from a namespace loaded by ``load_yaml_args`` (sections are flattened at load time, so
    the section name is accepted for call compatibility only; reference: yaml_arguments.py:403)."""
    return core_transformer_config_from_args(args)


def load_yaml(yaml_path: str, args=None):
    """A YAML file as an argument namespace on top of the parser's defaults (reference: yaml_arguments.py:442)."""
    base = args if args is not None else parse_args(argv=[])
    return load_yaml_args(yaml_path, base)
