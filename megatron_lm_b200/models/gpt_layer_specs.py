"""Layer specifications for the GPT family: which module fills each slot of a transformer layer.

The reference builds its layers from ``ModuleSpec`` trees and offers one tree per back end (Transformer Engine,
local PyTorch, Kitchen; megatron/core/models/gpt/gpt_layer_specs.py:72,:196,:362,:395,:499 and
moe_module_specs.py).  Here there is one back end - the sm_100a kernels of this library - so the Transformer-Engine
flavoured entry points return the same native tree; the functions and dataclasses keep the reference's names and
arguments so that model-provider code ports unchanged.  A spec is honoured, not ignored: ``TransformerLayer`` builds
every slot from it, so a user can swap the norm, the attention or the MLP of chosen layers for a class of their own
(constructed with those of ``config``, ``layer_number``, ``hidden_size``, ``causal`` that its signature names).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Union

from .spec_utils import ModuleSpec


@dataclass
class SelfAttentionSubmodules:
    linear_qkv: Any = None
    core_attention: Any = None
    linear_proj: Any = None
    q_layernorm: Any = None
    k_layernorm: Any = None


@dataclass
class MLPSubmodules:
    linear_fc1: Any = None
    linear_fc2: Any = None


@dataclass
class MoESubmodules:
    experts: Any = None
    shared_experts: Any = None


@dataclass
class TransformerLayerSubmodules:
    input_layernorm: Any = None
    self_attention: Any = None
    self_attn_bda: Any = None
    pre_cross_attn_layernorm: Any = None
    cross_attention: Any = None
    cross_attn_bda: Any = None
    pre_mlp_layernorm: Any = None
    mlp: Any = None
    mlp_bda: Any = None
    sharded_state_dict_keys_map: Dict[str, str] = field(default_factory=dict)


@dataclass
class TransformerBlockSubmodules:
    layer_specs: Optional[List[ModuleSpec]] = None
    layer_norm: Any = None


def _norm_class(normalization: Optional[str] = None):
    from .transformer import Norm
    return Norm


def get_mlp_module_spec(use_te: bool = True, num_experts: Optional[int] = None, moe_grouped_gemm: bool = False,
                        fp8: Optional[str] = None, moe_use_legacy_grouped_gemm: bool = False) -> ModuleSpec:
    """Dense MLP, or the MoE layer when ``num_experts`` is given (reference: gpt_layer_specs.py:362)."""
    from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
    from .transformer import MLP
    if num_experts is None:
        return ModuleSpec(module=MLP, submodules=MLPSubmodules(linear_fc1=ColumnParallelLinear,
                                                               linear_fc2=RowParallelLinear))
    return get_moe_module_spec(use_te=use_te, num_experts=num_experts, moe_grouped_gemm=moe_grouped_gemm)


def get_moe_module_spec(use_te: bool = True, num_experts: Optional[int] = None, moe_grouped_gemm: bool = False,
                        moe_use_legacy_grouped_gemm: bool = False) -> ModuleSpec:
    """reference: moe_module_specs.py:20"""
    from .moe import GroupedMLP, MoELayer, SequentialMLP, SharedExpertMLP
    experts = ModuleSpec(module=GroupedMLP if moe_grouped_gemm else SequentialMLP)
    return ModuleSpec(module=MoELayer, submodules=MoESubmodules(experts=experts,
                                                                shared_experts=ModuleSpec(module=SharedExpertMLP)))


def get_gpt_layer_local_spec(num_experts: Optional[int] = None, moe_grouped_gemm: bool = False,
                             qk_layernorm: bool = False, multi_latent_attention: bool = False, fp8: Optional[str] = None,
                             moe_use_legacy_grouped_gemm: bool = False, normalization: Optional[str] = None,
                             qk_l2_norm: bool = False, use_kitchen: bool = False) -> ModuleSpec:
    """One decoder layer (reference: gpt_layer_specs.py:196)."""
    from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
    from .transformer import IdentityOp, L2Norm, SelfAttention, TransformerLayer
    norm = _norm_class(normalization)
    if multi_latent_attention:
        from .mla import MLASelfAttention
        attn_cls = MLASelfAttention
    else:
        attn_cls = SelfAttention
    qk = L2Norm if qk_l2_norm else (norm if qk_layernorm else IdentityOp)
    attn = ModuleSpec(module=attn_cls, params={"attn_mask_type": "causal"},
                      submodules=SelfAttentionSubmodules(linear_qkv=ColumnParallelLinear, core_attention="flash",
                                                         linear_proj=RowParallelLinear, q_layernorm=qk, k_layernorm=qk))
    return ModuleSpec(module=TransformerLayer, submodules=TransformerLayerSubmodules(
        input_layernorm=norm, self_attention=attn, self_attn_bda="bias_dropout_add", pre_mlp_layernorm=norm,
        mlp=get_mlp_module_spec(False, num_experts, moe_grouped_gemm), mlp_bda="bias_dropout_add",
        sharded_state_dict_keys_map={"input_layernorm.": "self_attention.linear_qkv.layer_norm_",
                                     "pre_mlp_layernorm.": "mlp.linear_fc1.layer_norm_"}))


def get_gpt_layer_with_transformer_engine_spec(num_experts: Optional[int] = None, moe_grouped_gemm: bool = False,
                                               qk_layernorm: bool = False, multi_latent_attention: bool = False,
                                               fp8: Optional[str] = None, moe_use_legacy_grouped_gemm: bool = False,
                                               qk_l2_norm: bool = False, use_te_op_fuser: bool = False,
                                               use_kitchen: bool = False) -> ModuleSpec:
    """The fused-kernel layer.  The reference gets its fused kernels from Transformer Engine
    (gpt_layer_specs.py:72); this library's own kernels play that part, so the tree is the native one."""
    return get_gpt_layer_local_spec(num_experts, moe_grouped_gemm, qk_layernorm, multi_latent_attention, fp8,
                                    moe_use_legacy_grouped_gemm, None, qk_l2_norm, use_kitchen)


def get_gpt_decoder_block_spec(config, use_transformer_engine: bool = True, normalization: Optional[str] = None,
                               qk_l2_norm: bool = False, vp_stage: Optional[int] = None) -> TransformerBlockSubmodules:
    """Per-layer specs of the whole decoder: dense or MoE by ``config.moe_layer_freq`` (reference:
    gpt_layer_specs.py:395).  The list covers every layer of the model; a pipeline stage takes its slice."""
    dense = get_gpt_layer_local_spec(None, False, config.qk_layernorm, getattr(config, "multi_latent_attention", False),
                                     normalization=normalization, qk_l2_norm=qk_l2_norm)
    moe = get_gpt_layer_local_spec(config.num_moe_experts, config.moe_grouped_gemm, config.qk_layernorm,
                                   getattr(config, "multi_latent_attention", False), normalization=normalization,
                                   qk_l2_norm=qk_l2_norm) if config.num_moe_experts else dense
    pattern = config.moe_layer_pattern()
    return TransformerBlockSubmodules(layer_specs=[moe if pattern[i] else dense for i in range(config.num_layers)],
                                      layer_norm=_norm_class(normalization))


def get_gpt_mtp_block_spec(config, spec: Union[TransformerBlockSubmodules, ModuleSpec],
                           use_transformer_engine: bool = True, vp_stage: Optional[int] = None) -> Optional[ModuleSpec]:
    """Multi-token-prediction block: one transformer layer spec per predicted offset (reference:
    gpt_layer_specs.py:499).  None when the config predicts one token."""
    if not config.mtp_num_layers:
        return None
    from .mtp import MultiTokenPredictionBlock
    layer = spec.layer_specs[-1] if isinstance(spec, TransformerBlockSubmodules) else spec
    return ModuleSpec(module=MultiTokenPredictionBlock, submodules=[layer] * config.mtp_num_layers)


def layer_spec_is_moe(spec: Optional[ModuleSpec]) -> Optional[bool]:
    """Whether a layer spec puts a mixture-of-experts layer in the MLP slot (None: the spec does not say)."""
    if spec is None or spec.submodules is None or getattr(spec.submodules, "mlp", None) is None:
        return None
    from .moe import MoELayer
    mlp = spec.submodules.mlp
    cls = mlp.module if isinstance(mlp, ModuleSpec) else mlp
    return isinstance(cls, type) and issubclass(cls, MoELayer)
