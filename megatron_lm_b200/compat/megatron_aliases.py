"""``install()`` registers this library's modules under the reference's import paths, so that

    from megatron.core import parallel_state, tensor_parallel
    from megatron.core.models.gpt import GPTModel
    from megatron.core.transformer.transformer_config import TransformerConfig
    from megatron.core.pipeline_parallel import get_forward_backward_func
    from megatron.training import get_args, pretrain

resolve to the native implementations.  Nothing is aliased until ``install()`` is called, no file of this repository
is named ``megatron``, and ``install()`` refuses to run when a real ``megatron`` package is already imported - the
unmodified reference can therefore live on the same machine (the benchmark's reference arm imports it).

The table below is the map; a left-hand path that is a package in the reference (``megatron.core.models.gpt``)
becomes a synthetic module that re-exports the listed names.
"""
from __future__ import annotations

import importlib
import sys
import types
from typing import Dict, List, Tuple, Union

P = "megatron_lm_b200"

# alias path -> module path (whole-module alias) or list of (module path, [names]) to re-export
_MAP: Dict[str, Union[str, List[Tuple[str, List[str]]]]] = {
    "megatron.core.parallel_state": f"{P}.parallel.state",
    "megatron.core.process_groups_config": f"{P}.parallel.process_groups_config",
    "megatron.core.hyper_comm_grid": f"{P}.parallel.hyper_comm_grid",
    "megatron.core.tensor_parallel": [
        (f"{P}.parallel.layers", ["ColumnParallelLinear", "RowParallelLinear", "VocabParallelEmbedding",
                                  "set_tensor_model_parallel_attributes"]),
        (f"{P}.parallel.mappings", ["copy_to_tensor_model_parallel_region", "reduce_from_tensor_model_parallel_region",
                                    "scatter_to_tensor_model_parallel_region", "gather_from_tensor_model_parallel_region",
                                    "scatter_to_sequence_parallel_region", "gather_from_sequence_parallel_region",
                                    "reduce_scatter_to_sequence_parallel_region", "all_to_all", "all_to_all_sp2hp",
                                    "all_to_all_hp2sp"]),
        (f"{P}.parallel.random", ["get_cuda_rng_tracker", "model_parallel_cuda_manual_seed", "checkpoint",
                                  "CheckpointWithoutOutput", "get_expert_parallel_rng_tracker_name",
                                  "get_data_parallel_rng_tracker_name"]),
        (f"{P}.training.batch", ["broadcast_data"]),
    ],
    "megatron.core.tensor_parallel.layers": f"{P}.parallel.layers",
    "megatron.core.tensor_parallel.mappings": f"{P}.parallel.mappings",
    "megatron.core.tensor_parallel.random": f"{P}.parallel.random",
    "megatron.core.pipeline_parallel": [(f"{P}.parallel.schedules", ["get_forward_backward_func"])],
    "megatron.core.pipeline_parallel.schedules": f"{P}.parallel.schedules",
    "megatron.core.pipeline_parallel.p2p_communication": f"{P}.parallel.p2p",
    "megatron.core.distributed": [
        (f"{P}.parallel.ddp", ["DistributedDataParallel"]),
        (f"{P}.config", ["DistributedDataParallelConfig"]),
        (f"{P}.parallel.finalize_model_grads", ["finalize_model_grads"]),
        (f"{P}.parallel.fsdp", ["FullyShardedDataParallel", "TorchFullyShardedDataParallel"]),
    ],
    "megatron.core.optimizer": [
        (f"{P}.config", ["OptimizerConfig"]),
        (f"{P}.optimizer.optimizer", ["get_megatron_optimizer", "MixedPrecisionOptimizer", "ChainedOptimizer"]),
    ],
    "megatron.core.optimizer_param_scheduler": f"{P}.optimizer.scheduler",
    "megatron.core.num_microbatches_calculator": f"{P}.utils.num_microbatches_calculator",
    "megatron.core.transformer": [(f"{P}.config", ["TransformerConfig", "MLATransformerConfig"]),
                                  (f"{P}.models.spec_utils", ["ModuleSpec", "build_module"]),
                                  (f"{P}.models.module", ["MegatronModule"])],
    "megatron.core.transformer.transformer_config": [(f"{P}.config", ["TransformerConfig", "MLATransformerConfig"])],
    "megatron.core.transformer.spec_utils": f"{P}.models.spec_utils",
    "megatron.core.transformer.module": f"{P}.models.module",
    "megatron.core.transformer.enums": f"{P}.models.enums",
    "megatron.core.transformer.transformer_layer": [(f"{P}.models.transformer", ["TransformerLayer"]),
                                                    (f"{P}.models.gpt_layer_specs", ["TransformerLayerSubmodules"])],
    "megatron.core.transformer.transformer_block": [(f"{P}.models.transformer", ["TransformerBlock"]),
                                                    (f"{P}.models.gpt_layer_specs", ["TransformerBlockSubmodules"])],
    "megatron.core.transformer.moe.moe_layer": [(f"{P}.models.moe", ["MoELayer"])],
    "megatron.core.transformer.moe.router": [(f"{P}.models.moe", ["TopKRouter"])],
    "megatron.core.transformer.moe.moe_utils": f"{P}.models.moe",
    "megatron.core.models.gpt": [(f"{P}.models.gpt", ["GPTModel"])],
    "megatron.core.models.gpt.gpt_model": [(f"{P}.models.gpt", ["GPTModel"])],
    "megatron.core.models.gpt.gpt_layer_specs": f"{P}.models.gpt_layer_specs",
    "megatron.core.models.bert.bert_model": [(f"{P}.models.bert", ["BertModel"])],
    "megatron.core.models.T5.t5_model": [(f"{P}.models.t5", ["T5Model"])],
    "megatron.core.models.mamba.mamba_model": [(f"{P}.models.mamba", ["MambaModel"])],
    "megatron.core.models.backends": f"{P}.models.backends",
    "megatron.core.extensions.transformer_engine": f"{P}.extensions.transformer_engine",
    "megatron.core.dist_checkpointing": f"{P}.checkpoint.sharded",
    "megatron.core.datasets.indexed_dataset": f"{P}.data.indexed_dataset",
    "megatron.core.datasets.gpt_dataset": f"{P}.data.gpt_dataset",
    "megatron.core.rerun_state_machine": f"{P}.training.resilience",
    "megatron.core.packed_seq_params": f"{P}.packed_seq_params",
    "megatron.core.fp8_utils": f"{P}.fp8_utils",
    "megatron.core.activations": f"{P}.activations",
    "megatron.core.timers": f"{P}.utils.timers",
    "megatron.core.energy_monitor": f"{P}.utils.energy_monitor",
    "megatron.core.config_logger": f"{P}.utils.config_logger",
    "megatron.core.inference.engines": [(f"{P}.inference.engine", ["StaticInferenceEngine", "DynamicInferenceEngine"])],
    "megatron.core.inference.sampling_params": [(f"{P}.inference.engine", ["SamplingParams"])],
    "megatron.training": [
        (f"{P}.training.global_vars", ["get_args", "get_timers", "get_tokenizer", "get_tensorboard_writer",
                                       "get_wandb_writer"]),
        (f"{P}.training.pretrain", ["pretrain", "initialize_megatron"]),
    ],
    "megatron.training.arguments": f"{P}.training.arguments",
    "megatron.training.checkpointing": f"{P}.training.checkpointing",
    "megatron.training.global_vars": f"{P}.training.global_vars",
    "megatron.training.training": f"{P}.training.pretrain",
    "megatron.training.tokenizer": f"{P}.data.tokenizer",
    "megatron.training.yaml_arguments": [(f"{P}.training.arguments", ["validate_yaml", "core_transformer_config_from_yaml",
                                                                      "load_yaml"])],
    "megatron.core.dist_checkpointing.tensor_aware_state_dict": f"{P}.checkpoint.tensor_aware",
    "megatron.core.datasets.multimodal_dataset": f"{P}.data.multimodal_dataset",
    "megatron.core.datasets.object_storage_utils": f"{P}.data.object_storage",
    "megatron.core.transformer.moe.upcycling_utils": f"{P}.models.upcycling",
    "megatron.core.transformer.heterogeneous.heterogeneous_config": f"{P}.models.heterogeneous",
    "megatron.core.models.vision.clip_vit_model": [(f"{P}.models.vision", ["CLIPViTModel", "get_num_image_embeddings"])],
    "megatron.core.models.multimodal.llava_model": [(f"{P}.models.multimodal", ["LLaVAModel"])],
    "megatron.core.export.trtllm.trtllm_helper": [(f"{P}.export.trtllm", ["TRTLLMHelper"])],
    "megatron.core.quantization.quant_config": f"{P}.post_training.quant_config",
    "megatron.post_training.arguments": f"{P}.post_training.arguments",
    "megatron.post_training.checkpointing": f"{P}.post_training.checkpointing",
    "megatron.post_training.algos.distillation": f"{P}.post_training.distillation",
    "megatron.post_training.loss_func": [(f"{P}.post_training.distillation", ["distillation_loss_func", "masked_token_mean"])],
}
_PARENTS = ["megatron", "megatron.core", "megatron.core.models", "megatron.core.models.bert", "megatron.core.models.T5",
            "megatron.core.models.mamba", "megatron.core.transformer.moe", "megatron.core.extensions",
            "megatron.core.datasets", "megatron.core.inference", "megatron.core.transformer.heterogeneous",
            "megatron.core.models.vision", "megatron.core.models.multimodal", "megatron.core.export",
            "megatron.core.export.trtllm", "megatron.core.quantization", "megatron.post_training",
            "megatron.post_training.algos"]

_installed: List[str] = []


def install() -> List[str]:
    """Register the aliases; returns the alias paths.  Raises if a package named ``megatron`` that is not made of
    these aliases is already imported."""
    if _installed:
        return list(_installed)
    existing = sys.modules.get("megatron")
    if existing is not None and not getattr(existing, "__mlb_alias__", False):
        raise RuntimeError("a real 'megatron' package is already imported; aliases would shadow it")

    def synthetic(name):
        m = sys.modules.get(name)
        if m is None:
            m = types.ModuleType(name)
            m.__path__ = []                     # a package, so that sub-module imports are attempted
            m.__mlb_alias__ = True
            sys.modules[name] = m
            _installed.append(name)
        return m

    def attach(name, module):
        parent, _, leaf = name.rpartition(".")
        if parent:
            setattr(synthetic(parent) if parent not in sys.modules else sys.modules[parent], leaf, module)

    for name in _PARENTS:
        attach(name, synthetic(name))
    for alias, target in sorted(_MAP.items(), key=lambda kv: kv[0].count(".")):
        if isinstance(target, str):
            real = importlib.import_module(target)
            if alias in sys.modules and getattr(sys.modules[alias], "__mlb_alias__", False):
                # a synthetic parent created earlier: keep it a package, fill it with the module's names
                holder = sys.modules[alias]
                for k, v in vars(real).items():
                    if not k.startswith("__"):
                        setattr(holder, k, v)
                attach(alias, holder)
                continue
            sys.modules[alias] = real
            _installed.append(alias)
            attach(alias, real)
        else:
            holder = synthetic(alias)
            for mod_path, names in target:
                real = importlib.import_module(mod_path)
                for n in names:
                    setattr(holder, n, getattr(real, n))
            attach(alias, holder)
    return list(_installed)


def uninstall() -> None:
    for name in _installed:
        sys.modules.pop(name, None)
    _installed.clear()
