"""Per-layer ("heterogeneous", NAS-style) transformer configurations.

Reference: megatron/core/transformer/heterogeneous/heterogeneous_config.py (``HeterogeneousTransformerConfig``
:127, block-config JSON with per-layer ``attention`` {no_op, replace_with_linear, n_heads_in_group} and
``ffn`` {no_op, replace_with_linear, ffn_mult / intermediate_size}) and linear_replacements.py.
``per_layer_configs`` yields one ``TransformerConfig`` copy per layer; ``HeterogeneousLayer`` builds a layer
whose attention / MLP may be absent or replaced by a single linear map.
"""
from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn

from ..config import TransformerConfig
from ..ops import core as ops
from ..parallel.layers import ColumnParallelLinear
from .transformer import MLP, Norm, SelfAttention


@dataclass
class BlockSpec:
    attn_no_op: bool = False
    attn_linear: bool = False
    num_query_groups: Optional[int] = None
    mlp_no_op: bool = False
    mlp_linear: bool = False
    ffn_hidden_size: Optional[int] = None


def _ffn_mult_to_size(mult: float, hidden: int, multiple: int = 256) -> int:
    n = int(2 * mult * hidden / 3)
    return (n + multiple - 1) // multiple * multiple


def parse_block_configs(encoded: str, config: TransformerConfig) -> List[BlockSpec]:
    """``encoded``: JSON text (or a path to a JSON file) with a ``block_configs`` list."""
    try:
        cfg = json.loads(encoded)
    except json.JSONDecodeError:
        with open(encoded) as f:
            cfg = json.load(f)
    specs = []
    for b in cfg["block_configs"]:
        a, f = b.get("attention", {}), b.get("ffn", {})
        s = BlockSpec(attn_no_op=bool(a.get("no_op")), attn_linear=bool(a.get("replace_with_linear")),
                      mlp_no_op=bool(f.get("no_op")), mlp_linear=bool(f.get("replace_with_linear")))
        if a.get("n_heads_in_group"):
            s.num_query_groups = config.num_attention_heads // int(a["n_heads_in_group"])
        if f.get("intermediate_size"):
            s.ffn_hidden_size = int(f["intermediate_size"])
        elif f.get("ffn_mult"):
            s.ffn_hidden_size = _ffn_mult_to_size(float(f["ffn_mult"]), config.hidden_size)
        specs.append(s)
    if len(specs) != config.num_layers:
        raise ValueError("block_configs must list one entry per layer")
    return specs


def per_layer_configs(config: TransformerConfig, specs: List[BlockSpec]) -> List[TransformerConfig]:
    out = []
    for s in specs:
        c = copy.copy(config)
        if s.num_query_groups is not None:
            c.num_query_groups = s.num_query_groups
        if s.ffn_hidden_size is not None:
            c.ffn_hidden_size = s.ffn_hidden_size
        out.append(c)
    return out


class _LinearReplacement(nn.Module):
    """norm -> one hidden x hidden linear, standing in for a whole attention or MLP block."""

    def __init__(self, config):
        super().__init__()
        self.linear = ColumnParallelLinear(config.hidden_size, config.hidden_size, config=config,
                                           init_method=config.init_method, bias=False, gather_output=True,
                                           disable_sp_gather=True)

    def forward(self, x, **_):
        return self.linear(x)


class HeterogeneousLayer(nn.Module):
    def __init__(self, config: TransformerConfig, spec: BlockSpec, layer_number: int):
        super().__init__()
        self.config, self.spec, self.layer_number = config, spec, layer_number
        if not spec.attn_no_op:
            self.input_layernorm = Norm(config, config.hidden_size)
            self.self_attention = _LinearReplacement(config) if spec.attn_linear else SelfAttention(config, layer_number)
        if not spec.mlp_no_op:
            self.pre_mlp_layernorm = Norm(config, config.hidden_size)
            self.mlp = _LinearReplacement(config) if spec.mlp_linear else MLP(config)
        self.p = config.hidden_dropout

    def forward(self, h, rotary=None, inference_context=None, **_):
        if not self.spec.attn_no_op:
            if self.spec.attn_linear:
                out, bias = self.self_attention(self.input_layernorm(h))
            else:
                out, bias = self.self_attention(self.input_layernorm(h), rotary=rotary, inference_context=inference_context)
            h = ops.bias_dropout_add(out, bias, h, self.p, self.training)
        if not self.spec.mlp_no_op:
            out, bias = self.mlp(self.pre_mlp_layernorm(h))
            h = ops.bias_dropout_add(out, bias, h, self.p, self.training)
        return h


def build_heterogeneous_layers(config: TransformerConfig, encoded_block_configs: str, offset: int = 0,
                               count: Optional[int] = None) -> nn.ModuleList:
    specs = parse_block_configs(encoded_block_configs, config)
    cfgs = per_layer_configs(config, specs)
    count = len(specs) - offset if count is None else count
    return nn.ModuleList([HeterogeneousLayer(cfgs[offset + i], specs[offset + i], offset + i + 1) for i in range(count)])
