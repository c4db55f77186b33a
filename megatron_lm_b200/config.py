"""Configuration dataclasses.

Field names follow the reference library so that launch scripts and user code
translate one to one (reference: megatron/core/model_parallel_config.py:10,
megatron/core/transformer/transformer_config.py:33,
megatron/core/optimizer/optimizer_config.py:12,
megatron/core/distributed/distributed_data_parallel_config.py:8).  The
validation in ``__post_init__`` keeps the combination rules of the reference
(transformer_config.py:650-1336) that matter for the features built here.
"""
from __future__ import annotations

import math
import dataclasses
from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional, Tuple, Union

import torch


@dataclass
class ModelParallelConfig:
    # --- model parallelism
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_comm_backend: Optional[str] = None
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    sequence_parallel: bool = False
    context_parallel_size: int = 1
    hierarchical_context_parallel_sizes: Optional[List[int]] = None
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Optional[int] = None
    moe_extended_tp: bool = False
    # --- initialisation
    perform_initialization: bool = True
    use_cpu_initialization: bool = False
    # --- precision
    fp16: bool = False
    bf16: bool = False
    params_dtype: torch.dtype = torch.float32
    timers: Any = None
    # --- callbacks installed by the training loop and called by the schedules
    finalize_model_grads_func: Optional[Callable] = None
    grad_scale_func: Optional[Callable] = None
    no_sync_func: Optional[Callable] = None
    grad_sync_func: Optional[Callable] = None
    param_sync_func: Optional[Callable] = None
    deterministic_mode: bool = False
    enable_autocast: bool = False
    autocast_dtype: Optional[torch.dtype] = None
    num_microbatches_with_partial_activation_checkpoints: Optional[int] = None
    # --- optimisations
    gradient_accumulation_fusion: bool = True
    async_tensor_model_parallel_allreduce: bool = False
    use_te_rng_tracker: bool = False
    # tp_comm_overlap selects the fused peer-memory all-gather->GEMM and
    # GEMM->reduce-scatter kernels (the reference used userbuffers for this).
    tp_comm_overlap: bool = False
    tp_comm_bulk_wgrad: bool = True
    tp_comm_bulk_dgrad: bool = True
    tp_comm_overlap_ag: bool = True
    tp_comm_overlap_rs: bool = True
    tp_comm_overlap_rs_dgrad: bool = False
    tp_comm_split_ag: bool = True
    tp_comm_atomic_ag: bool = False
    tp_comm_split_rs: bool = True
    tp_comm_atomic_rs: bool = False
    cross_entropy_loss_fusion: bool = True
    cross_entropy_fusion_impl: str = "native"
    tp_comm_overlap_disable_qkv: bool = False
    tp_comm_overlap_disable_fc1: bool = False
    tp_comm_bootstrap_backend: str = "nccl"
    overlap_moe_expert_parallel_comm: bool = False
    delay_wgrad_compute: bool = False
    # --- pipeline
    pipeline_dtype: Optional[torch.dtype] = None
    variable_seq_lengths: bool = False
    overlap_p2p_comm: bool = False
    batch_p2p_comm: bool = True
    batch_p2p_sync: bool = True
    use_ring_exchange_p2p: bool = False
    deallocate_pipeline_outputs: bool = False
    defer_embedding_wgrad_compute: bool = False
    wgrad_deferral_limit: int = 0
    overlap_p2p_comm_warmup_flush: bool = False
    microbatch_group_size_per_vp_stage: Optional[int] = None
    # --- cpu offload
    cpu_offloading: bool = False
    cpu_offloading_num_layers: int = 0
    _cpu_offloading_context: Any = None
    cpu_offloading_activations: bool = True
    cpu_offloading_weights: bool = False
    barrier_with_L1_time: bool = True

    def __post_init__(self):
        if self.sequence_parallel and self.tensor_model_parallel_size <= 1:
            raise ValueError("sequence_parallel requires tensor_model_parallel_size > 1")
        if self.expert_tensor_parallel_size is None:
            self.expert_tensor_parallel_size = self.tensor_model_parallel_size
        if self.pipeline_model_parallel_size > 1 and self.pipeline_dtype is None:
            self.pipeline_dtype = self.params_dtype
        if self.autocast_dtype is None:
            self.autocast_dtype = self.params_dtype
        if self.defer_embedding_wgrad_compute and self.pipeline_model_parallel_size == 1:
            raise ValueError("defer_embedding_wgrad_compute needs pipeline parallelism")
        if self.virtual_pipeline_model_parallel_size is not None and self.virtual_pipeline_model_parallel_size > 1:
            if self.pipeline_model_parallel_size <= 1:
                raise ValueError("interleaved schedule needs pipeline_model_parallel_size > 1")
        if self.microbatch_group_size_per_vp_stage is None:
            self.microbatch_group_size_per_vp_stage = self.pipeline_model_parallel_size
        if self.overlap_p2p_comm_warmup_flush and not self.overlap_p2p_comm:
            raise ValueError("overlap_p2p_comm_warmup_flush requires overlap_p2p_comm")


# Fields of the reference's configuration that this framework accepts (so configurations carry over) but does not
# implement, and that would change the numerics, the model or the memory plan if they were honoured: asking for one
# of them stops the construction of the configuration instead of silently building something else.  Fields that
# only pick between implementations of the same mathematics (fusion switches, library back ends, CUDA-graph and
# communication-overlap tuning knobs) are accepted without effect: there is one implementation here.
UNSUPPORTED_FIELDS = {
    "fp8_dot_product_attention": "attention runs in bf16 / fp16",
    "fp8_multi_head_attention": "attention runs in bf16 / fp16",
    "init_model_with_meta_device": "parameters are created on their device",
    "enable_cuda_graph": "the training loop captures no graphs; wrap single modules with utils.cuda_graphs.GraphedModule "
                         "or a whole step with FullIterationGraph from a hand-written loop",
    "external_cuda_graph": "the training loop captures no graphs",
    "use_kitchen": "the Kitchen quantisation back end is not built",
    "quant_recipe": "per-layer quantisation recipes are not built",
    "heterogeneous_block_specs": "build heterogeneous models through models.heterogeneous",
}


def check_unsupported_fields(cfg) -> None:
    defaults = {f.name: f.default for f in dataclasses.fields(type(cfg)) if f.default is not dataclasses.MISSING}
    for name, why in UNSUPPORTED_FIELDS.items():
        if not hasattr(cfg, name):
            continue
        v = getattr(cfg, name)
        d = defaults.get(name)
        if v == d or (v in (None, False, 0) and d in (None, False, 0)):
            continue
        raise ValueError(f"TransformerConfig.{name} = {v!r} is not supported: {why}")


def init_method_normal(sigma: float) -> Callable:
    def init_(t):
        return torch.nn.init.normal_(t, mean=0.0, std=sigma)
    return init_


def scaled_init_method_normal(sigma: float, num_layers: int, multiplier: float = 2.0) -> Callable:
    std = sigma / math.sqrt(multiplier * num_layers)

    def init_(t):
        return torch.nn.init.normal_(t, mean=0.0, std=std)
    return init_


@dataclass
class TransformerConfig(ModelParallelConfig):
    # --- architecture
    num_layers: int = 0
    mtp_num_layers: Optional[int] = None
    mtp_loss_scaling_factor: Optional[float] = None
    num_layers_in_first_pipeline_stage: Optional[int] = None
    num_layers_in_last_pipeline_stage: Optional[int] = None
    pipeline_model_parallel_layout: Optional[Union[str, list]] = None
    account_for_embedding_in_pipeline_split: bool = False
    account_for_loss_in_pipeline_split: bool = False
    hidden_size: int = 0
    num_attention_heads: int = 0
    attention_backend: str = "auto"
    softmax_scale: Optional[float] = None
    num_query_groups: Optional[int] = None
    ffn_hidden_size: Optional[int] = None
    kv_channels: Optional[int] = None
    hidden_dropout: float = 0.1
    attention_dropout: float = 0.1
    fp32_residual_connection: bool = False
    apply_residual_connection_post_layernorm: bool = False
    layernorm_epsilon: float = 1e-5
    layernorm_zero_centered_gamma: bool = False
    add_bias_linear: bool = True
    add_qkv_bias: bool = False
    gated_linear_unit: bool = False
    activation_func: Union[str, Callable] = "gelu"
    activation_func_fp8_input_store: bool = False
    num_moe_experts: Optional[int] = None
    rotary_interleaved: bool = False
    window_size: Optional[Tuple[int, int]] = None
    normalization: str = "LayerNorm"
    qk_layernorm: bool = False
    qk_l2_norm: bool = False          # parameter-free L2 normalisation of queries and keys (Llama-4 style)
    test_mode: bool = False
    calculate_per_token_loss: bool = False
    multi_latent_attention: bool = False
    no_rope_freq: Optional[Union[int, List[int]]] = None
    moe_deepep_num_sms: int = 20
    # --- position embedding (the reference keeps these on the model; kept
    # here too so one object describes a model)
    position_embedding_type: str = "learned_absolute"
    rotary_percent: float = 1.0
    rotary_base: float = 10000.0
    rotary_scaling_factor: Optional[float] = None
    max_position_embeddings: int = 2048
    share_embeddings_and_output_weights: bool = True
    # --- init
    init_method: Optional[Callable] = None
    output_layer_init_method: Optional[Callable] = None
    init_method_std: float = 0.02
    embedding_init_method: Optional[Callable] = None
    embedding_init_method_std: Optional[float] = None
    init_model_with_meta_device: bool = False
    # --- mixed precision
    apply_query_key_layer_scaling: bool = False
    attention_softmax_in_fp32: bool = True
    disable_bf16_reduced_precision_matmul: bool = False
    # --- fusion switches (every fused op here is the only implementation;
    # the flags are accepted for launch-script compatibility)
    bias_activation_fusion: bool = True
    masked_softmax_fusion: bool = True
    persist_layer_norm: bool = True
    memory_efficient_layer_norm: bool = False
    bias_dropout_fusion: bool = True
    apply_rope_fusion: bool = True
    use_fused_weighted_squared_relu: bool = False
    # --- activation recompute
    recompute_granularity: Optional[str] = None
    recompute_method: Optional[str] = None
    recompute_num_layers: Optional[int] = None
    distribute_saved_activations: bool = False
    recompute_modules: Optional[List[str]] = None
    # --- fp8
    fp8: Optional[str] = None
    fp8_recipe: Optional[str] = "delayed"
    fp8_param: bool = False
    fp8_margin: int = 0
    fp8_interval: int = 1
    fp8_amax_history_len: int = 1
    fp8_amax_compute_algo: str = "most_recent"
    fp8_wgrad: bool = True
    fp8_dot_product_attention: bool = False
    fp8_multi_head_attention: bool = False
    tp_only_amax_red: bool = False
    first_last_layers_bf16: bool = False
    num_layers_at_start_in_bf16: int = 1
    num_layers_at_end_in_bf16: int = 1
    use_kitchen: bool = False
    # --- MoE
    moe_shared_expert_intermediate_size: Optional[int] = None
    moe_shared_expert_overlap: bool = False
    moe_layer_freq: Union[int, List[int]] = 1
    moe_ffn_hidden_size: Optional[int] = None
    moe_router_load_balancing_type: str = "aux_loss"
    moe_router_topk: int = 2
    moe_router_topk_limited_devices: Optional[int] = None
    moe_router_padding_for_fp8: bool = False
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    moe_router_pre_softmax: bool = False
    moe_router_topk_scaling_factor: Optional[float] = None
    moe_router_score_function: str = "softmax"
    moe_router_dtype: Optional[str] = None
    moe_router_enable_expert_bias: bool = False
    moe_router_bias_update_rate: float = 1e-3
    moe_router_force_load_balancing: bool = False
    moe_grouped_gemm: bool = False
    moe_use_legacy_grouped_gemm: bool = False
    moe_aux_loss_coeff: float = 0.0
    moe_z_loss_coeff: Optional[float] = None
    moe_input_jitter_eps: Optional[float] = None
    moe_token_dropping: bool = False
    moe_token_dispatcher_type: str = "allgather"
    moe_enable_deepep: bool = False
    moe_per_layer_logging: bool = False
    moe_expert_capacity_factor: Optional[float] = None
    moe_pad_expert_input_to_capacity: bool = False
    moe_token_drop_policy: str = "probs"
    moe_layer_recompute: bool = False
    moe_permute_fusion: bool = False
    moe_apply_probs_on_input: bool = False
    # --- context parallel
    cp_comm_type: Optional[Union[str, List[str]]] = None
    # --- cuda graphs
    enable_cuda_graph: bool = False
    cuda_graph_use_single_mempool: bool = False
    cuda_graph_retain_backward_graph: bool = False
    cuda_graph_warmup_steps: int = 3
    external_cuda_graph: bool = False
    cuda_graph_scope: str = "full"
    # --- misc
    clone_scatter_output_in_embedding: bool = True
    disable_parameter_transpose_cache: bool = False
    config_logger_dir: str = ""
    flash_decode: bool = False
    inference_rng_tracker: bool = False
    symmetric_ar_type: Optional[str] = None
    mrope_section: Optional[List[int]] = None
    is_hybrid_model: bool = False
    mamba_state_dim: int = 128
    mamba_head_dim: int = 64
    mamba_num_groups: int = 8
    mamba_num_heads: Optional[int] = None
    use_mamba_mem_eff_path: bool = True
    mlp_chunks_for_prefill: int = 1
    heterogeneous_block_specs: bool = False
    # per-layer block configuration (JSON text, the format of models/heterogeneous.py): layers may drop or replace
    # their attention / MLP and choose their own widths
    heterogeneous_layers_config_encoded_json: Optional[str] = None
    hetereogenous_dist_checkpoint: bool = False
    quant_recipe: Any = None

    def __post_init__(self):
        super().__post_init__()
        if self.fp16 and self.bf16:
            raise ValueError("fp16 and bf16 are mutually exclusive")
        if self.bf16 and self.params_dtype == torch.float32:
            self.params_dtype = torch.bfloat16
        if self.fp16 and self.params_dtype == torch.float32:
            self.params_dtype = torch.float16
        if self.num_layers <= 0 or self.hidden_size <= 0 or self.num_attention_heads <= 0:
            raise ValueError("num_layers, hidden_size and num_attention_heads must be set")
        check_unsupported_fields(self)
        if self.num_attention_heads % self.tensor_model_parallel_size != 0:
            raise ValueError(
                f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                f"tensor_model_parallel_size ({self.tensor_model_parallel_size})")
        if self.ffn_hidden_size is None:
            self.ffn_hidden_size = 4 * self.hidden_size
        if self.kv_channels is None:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        if self.num_query_groups % self.tensor_model_parallel_size != 0 and \
                self.tensor_model_parallel_size % self.num_query_groups != 0:
            raise ValueError("num_query_groups must divide or be divisible by the TP size")
        if self.num_attention_heads % self.num_query_groups != 0:
            raise ValueError("num_attention_heads must be a multiple of num_query_groups")
        if self.apply_query_key_layer_scaling:
            self.attention_softmax_in_fp32 = True
        if self.expert_model_parallel_size > 1 and self.num_moe_experts is None:
            raise ValueError("num_moe_experts must be set with expert parallelism")
        if self.num_moe_experts is not None:
            if self.num_moe_experts <= 0:
                raise ValueError("num_moe_experts must be positive")
            if self.num_moe_experts % self.expert_model_parallel_size != 0:
                raise ValueError("num_moe_experts must be divisible by expert_model_parallel_size")
            if self.moe_ffn_hidden_size is None:
                self.moe_ffn_hidden_size = self.ffn_hidden_size
        if self.delay_wgrad_compute and not self.overlap_moe_expert_parallel_comm:
            raise ValueError("delay_wgrad_compute needs overlap_moe_expert_parallel_comm (the schedule that runs the "
                             "postponed weight gradients)")
        if self.cpu_offloading:
            if self.cpu_offloading_weights:
                raise ValueError("cpu_offloading_weights is not supported: only activations are offloaded")
            if self.recompute_granularity == "full":
                raise ValueError("cpu_offloading and full activation recomputation exclude each other")
            if not 0 < self.cpu_offloading_num_layers <= self.num_layers:
                raise ValueError("cpu_offloading needs 0 < cpu_offloading_num_layers <= num_layers")
        if self.moe_router_topk_limited_devices and self.moe_router_num_groups is None:
            # older name of group-limited routing: one group per expert-parallel rank
            self.moe_router_num_groups = self.expert_model_parallel_size
            self.moe_router_group_topk = self.moe_router_topk_limited_devices
        if self.moe_apply_probs_on_input and self.moe_router_topk != 1:
            raise ValueError("moe_apply_probs_on_input needs moe_router_topk == 1")
        if self.moe_expert_capacity_factor is not None:
            if self.moe_expert_capacity_factor < 0:
                self.moe_expert_capacity_factor = None
            elif self.moe_router_load_balancing_type not in ("aux_loss", "seq_aux_loss", "none"):
                raise ValueError("capacity factor needs aux_loss / seq_aux_loss / none balancing")
        if self.moe_pad_expert_input_to_capacity and self.moe_expert_capacity_factor is None:
            raise ValueError("moe_pad_expert_input_to_capacity needs moe_expert_capacity_factor")
        if self.recompute_granularity is not None:
            if self.recompute_granularity not in ("full", "selective"):
                raise ValueError("recompute_granularity must be 'full' or 'selective'")
            if self.recompute_granularity == "full":
                if self.recompute_method not in ("uniform", "block"):
                    raise ValueError("full recompute needs recompute_method uniform|block")
                if self.recompute_num_layers is None:
                    self.recompute_num_layers = 1
            elif self.recompute_modules is None:
                self.recompute_modules = ["core_attn"]
        if self.recompute_modules is None:
            self.recompute_modules = []
        if self.distribute_saved_activations and self.sequence_parallel:
            raise ValueError("distribute_saved_activations is incompatible with sequence_parallel")
        if self.virtual_pipeline_model_parallel_size is not None and \
                self.pipeline_model_parallel_layout is None and \
                self.num_layers_in_first_pipeline_stage is None and \
                self.num_layers_in_last_pipeline_stage is None:
            per_stage = self.num_layers // self.pipeline_model_parallel_size
            if self.num_layers % self.pipeline_model_parallel_size != 0 or \
                    per_stage % self.virtual_pipeline_model_parallel_size != 0:
                raise ValueError("layers per pipeline stage must be divisible by the virtual pipeline size")
        if self.init_method is None:
            self.init_method = init_method_normal(self.init_method_std)
        if self.output_layer_init_method is None:
            self.output_layer_init_method = scaled_init_method_normal(self.init_method_std, self.num_layers)
        if self.embedding_init_method_std is None:
            self.embedding_init_method_std = self.init_method_std
        if self.embedding_init_method is None:
            self.embedding_init_method = init_method_normal(self.embedding_init_method_std)
        if self.fp8 is not None and self.fp8 not in ("e4m3", "hybrid"):
            raise ValueError("fp8 must be None, 'e4m3' or 'hybrid'")
        if self.cp_comm_type is None:
            self.cp_comm_type = "p2p"
        if self.moe_router_dtype not in (None, "fp32", "fp64"):
            raise ValueError("moe_router_dtype must be None, fp32 or fp64")
        if isinstance(self.moe_layer_freq, list) and len(self.moe_layer_freq) != self.num_layers:
            raise ValueError("moe_layer_freq list must have num_layers entries")

    # -- derived helpers -------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.kv_channels

    @property
    def is_moe(self) -> bool:
        return self.num_moe_experts is not None

    def moe_layer_pattern(self) -> List[int]:
        """1 where the layer's MLP is a mixture of experts (reference:
        megatron/core/models/gpt/gpt_layer_specs.py:395 decoder block spec)."""
        if not self.is_moe:
            return [0] * self.num_layers
        if isinstance(self.moe_layer_freq, int):
            return [1 if i % self.moe_layer_freq == 0 else 0 for i in range(self.num_layers)]
        return list(self.moe_layer_freq)


@dataclass
class MLATransformerConfig(TransformerConfig):
    """Multi-latent attention (reference: transformer_config.py:1340)."""
    multi_latent_attention: bool = True
    q_lora_rank: Optional[int] = 512
    kv_lora_rank: int = 512
    qk_head_dim: int = 128
    qk_pos_emb_head_dim: int = 64
    v_head_dim: int = 128
    normalization: str = "RMSNorm"
    rope_type: str = "yarn"
    rotary_base: float = 10000.0
    rotary_percent: float = 1.0
    rotary_scaling_factor: float = 40.0
    max_position_embeddings: int = 4096
    original_max_position_embeddings: int = 4096
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0


@dataclass
class OptimizerConfig:
    optimizer: str = "adam"
    lr: Optional[float] = None
    min_lr: Optional[float] = None
    decoupled_lr: Optional[float] = None
    decoupled_min_lr: Optional[float] = None
    weight_decay: float = 0.01
    fp8_recipe: Optional[str] = None
    fp16: bool = False
    bf16: bool = False
    reuse_grad_buf_for_mxfp8_param_ag: bool = False
    params_dtype: torch.dtype = torch.float32
    use_precision_aware_optimizer: bool = False
    store_param_remainders: bool = True
    main_grads_dtype: torch.dtype = torch.float32
    main_params_dtype: torch.dtype = torch.float32
    exp_avg_dtype: torch.dtype = torch.float32
    exp_avg_sq_dtype: torch.dtype = torch.float32
    loss_scale: Optional[float] = None
    initial_loss_scale: float = 2 ** 32
    min_loss_scale: float = 1.0
    loss_scale_window: float = 1000
    hysteresis: int = 2
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    sgd_momentum: float = 0.9
    use_distributed_optimizer: bool = False
    overlap_param_gather: bool = False
    overlap_param_gather_with_optimizer_step: bool = False
    optimizer_cpu_offload: bool = False
    optimizer_offload_fraction: float = 0.0
    use_torch_optimizer_for_cpu_offload: bool = False
    overlap_cpu_optimizer_d2h_h2d: bool = False
    pin_cpu_grads: bool = True
    pin_cpu_params: bool = True
    clip_grad: float = 1.0
    log_num_zeros_in_grad: bool = False
    barrier_with_L1_time: bool = False
    timers: Any = None
    config_logger_dir: str = ""

    def __post_init__(self):
        if self.optimizer not in ("adam", "sgd"):
            raise ValueError(f"unknown optimizer {self.optimizer}")
        if self.use_precision_aware_optimizer and not self.use_distributed_optimizer:
            raise ValueError("precision-aware optimizer needs the distributed optimizer")
        if self.optimizer_cpu_offload and not (0.0 <= self.optimizer_offload_fraction <= 1.0):
            raise ValueError("optimizer_offload_fraction must be in [0, 1]")


@dataclass
class DistributedDataParallelConfig:
    grad_reduce_in_fp32: bool = False
    overlap_grad_reduce: bool = False
    overlap_param_gather: bool = False
    align_param_gather: bool = False
    use_distributed_optimizer: bool = False
    num_distributed_optimizer_instances: int = 1
    check_for_nan_in_grad: bool = False
    check_for_large_grads: bool = False
    bucket_size: Optional[int] = None
    pad_buckets_for_high_nccl_busbw: bool = False
    average_in_collective: bool = False
    fp8_param_gather: bool = False
    reuse_grad_buf_for_mxfp8_param_ag: bool = False
    use_custom_fsdp: bool = False
    use_torch_fsdp2: bool = False
    torch_fsdp2_reshard_after_forward: bool = True
    data_parallel_sharding_strategy: str = "no_shard"
    gradient_reduce_div_fusion: bool = True
    suggested_communication_unit_size: Optional[int] = None
    preserve_fp32_weights: bool = True
    keep_fp8_transpose_cache_when_using_custom_fsdp: bool = False
    nccl_ub: bool = False
    # gradient reduce-scatter and parameter all-gather of the distributed optimizer as peer-memory kernels (pull-
    # reduce fused with scaling and norm, overlapped with the backward pass; AdamW storing its result into every
    # rank's parameter buffer).  On by default; it applies where it can - distributed optimizer, fp32 gradients, bf16
    # parameters, a data-parallel group of at most eight GPUs inside one node - and NCCL is used everywhere else.
    peer_memory_collectives: bool = True
    # thread blocks of one peer-memory gradient pull (it overlaps the backward pass, so it gets a small grid)
    peer_pull_blocks: int = 64
    # --ddp-num-buckets: split each buffer into this many buckets (overrides bucket_size)
    num_buckets: Optional[int] = None
    fsdp_double_buffer: bool = False

    def __post_init__(self):
        if self.data_parallel_sharding_strategy not in (
                "no_shard", "optim", "optim_grads", "optim_grads_params"):
            raise ValueError("bad data_parallel_sharding_strategy")
        if self.overlap_param_gather and not self.use_distributed_optimizer:
            raise ValueError("overlap_param_gather needs use_distributed_optimizer")
