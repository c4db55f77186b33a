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
    g.add_argument("--ec-device", default="auto", choices=["auto", "gpu", "cpu"],
                   help="where parity is computed and held: peer GPUs' memory (auto on NCCL jobs) or host memory")
    g = parser.add_argument_group(title="peer-memory kernels")
    g.add_argument("--peer-memory-collectives", action="store_true",
                   help="distributed optimizer: gradient reduce-scatter as a pull kernel over NVLink peer memory and "
                        "AdamW storing new weights into every rank's parameter buffer (single node)")
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
    # model sizes
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
    args.padded_vocab_size = getattr(args, "padded_vocab_size", None)
    args.consumed_train_samples = 0
    args.consumed_valid_samples = 0
    args.iteration = 0
    return args


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
        ("squared_relu" if getattr(args, "squared_relu", False) else "gelu"),
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
    kw["peer_memory_collectives"] = getattr(args, "peer_memory_collectives", False)
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
