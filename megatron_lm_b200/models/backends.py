"""Spec providers: the question "which class implements this building block?" asked by spec-building code
(reference: megatron/core/models/backends.py:26 BackendSpecProvider, :67 LocalSpecProvider;
extensions/transformer_engine_spec_provider.py:24 TESpecProvider; extensions/kitchen.py:1024).
Every provider answers with this library's modules; the Transformer-Engine-named provider answers with the
TE-named classes of ``extensions/transformer_engine.py``, which are the same kernels under the reference's names."""
from __future__ import annotations

from typing import Optional, Tuple


class BackendSpecProvider:
    def column_parallel_linear(self) -> type: raise NotImplementedError
    def row_parallel_linear(self) -> type: raise NotImplementedError
    def fuse_layernorm_and_linear(self) -> bool: raise NotImplementedError
    def column_parallel_layer_norm_linear(self) -> Optional[type]: raise NotImplementedError
    def layer_norm(self, rms_norm: bool = False, for_qk: bool = False) -> type: raise NotImplementedError
    def core_attention(self) -> type: raise NotImplementedError
    def grouped_mlp_modules(self, moe_use_grouped_gemm: bool, moe_use_legacy_grouped_gemm: bool) -> Tuple[type, object]:
        raise NotImplementedError
    def activation_func(self): raise NotImplementedError


class LocalSpecProvider(BackendSpecProvider):
    def column_parallel_linear(self):
        from ..parallel.layers import ColumnParallelLinear
        return ColumnParallelLinear

    def row_parallel_linear(self):
        from ..parallel.layers import RowParallelLinear
        return RowParallelLinear

    def fuse_layernorm_and_linear(self):
        return False

    def column_parallel_layer_norm_linear(self):
        return None

    def layer_norm(self, rms_norm: bool = False, for_qk: bool = False):
        from .transformer import Norm
        return Norm

    def core_attention(self):
        from ..extensions.transformer_engine import TEDotProductAttention
        return TEDotProductAttention

    def grouped_mlp_modules(self, moe_use_grouped_gemm: bool, moe_use_legacy_grouped_gemm: bool = False):
        from .gpt_layer_specs import MLPSubmodules
        from .moe import GroupedMLP, SequentialMLP
        if moe_use_grouped_gemm:
            return GroupedMLP, None
        return SequentialMLP, MLPSubmodules(linear_fc1=self.column_parallel_linear(),
                                            linear_fc2=self.row_parallel_linear())

    def activation_func(self):
        return None


class TESpecProvider(LocalSpecProvider):
    def column_parallel_linear(self):
        from ..extensions.transformer_engine import TEColumnParallelLinear
        return TEColumnParallelLinear

    def row_parallel_linear(self):
        from ..extensions.transformer_engine import TERowParallelLinear
        return TERowParallelLinear

    def fuse_layernorm_and_linear(self):
        return True

    def column_parallel_layer_norm_linear(self):
        from ..extensions.transformer_engine import TELayerNormColumnParallelLinear
        return TELayerNormColumnParallelLinear

    def layer_norm(self, rms_norm: bool = False, for_qk: bool = False):
        from ..extensions.transformer_engine import TENorm
        return TENorm


KitchenSpecProvider = LocalSpecProvider      # the quantised-linear back end of the reference: native FP8 path here
