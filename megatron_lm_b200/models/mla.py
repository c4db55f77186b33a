"""Multi-latent attention (DeepSeek-style low-rank Q / KV projections with a decoupled RoPE part).

Reference: megatron/core/transformer/multi_latent_attention.py (``MultiLatentAttention`` :65,
``MLASelfAttention`` :254) and models/common/embeddings/yarn_rotary_pos_embedding.py.

  q  = up_q(norm(down_q(x)))                     -> per head [qk_head_dim | qk_pos_emb_head_dim]
  kv = down_kv(x) = [latent (kv_lora_rank) | k_pos (shared by all heads)]
  k, v = up_kv(norm(latent))                     -> per head [qk_head_dim] , [v_head_dim]
  RoPE (YaRN-scaled) rotates only the positional parts; softmax scale carries mscale^2.

The down projections and their norms are replicated across tensor-parallel ranks (their gradients
are summed over the TP group when sequence parallelism splits the tokens); the up projections are
column-parallel over heads.  Query/key heads are 192 wide and value heads 128, which the flash
kernels of this package (64 / 128) do not cover, so the core product runs through
``torch.nn.functional.scaled_dot_product_attention``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import core as ops
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, _device
from ..parallel.mappings import gather_from_sequence_parallel_region


def _yarn_find_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def yarn_get_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


class YarnRotaryEmbedding(nn.Module):
    """cos/sin tables with YaRN frequency interpolation: high-frequency dims keep their wavelength,
    low-frequency dims are divided by ``scaling_factor``, with a linear ramp between the dims that make
    ``beta_fast`` and ``beta_slow`` rotations over the original context."""

    def __init__(self, dim: int, rotary_base: float = 10000.0, scaling_factor: float = 1.0,
                 original_max_position_embeddings: int = 4096, beta_fast: float = 32.0, beta_slow: float = 1.0,
                 mscale: float = 1.0, mscale_all_dim: float = 0.0):
        super().__init__()
        self.dim, self.base, self.factor = dim, rotary_base, scaling_factor
        self.orig, self.beta_fast, self.beta_slow = original_max_position_embeddings, beta_fast, beta_slow
        self.mscale, self.mscale_all_dim = mscale, mscale_all_dim
        self._cache = {}

    def _inv_freq(self, device):
        ex = torch.arange(0, self.dim, 2, dtype=torch.float32, device=device) / self.dim
        extra = 1.0 / (self.base ** ex)
        inter = 1.0 / (self.factor * self.base ** ex)
        low = max(math.floor(_yarn_find_dim(self.beta_fast, self.dim, self.base, self.orig)), 0)
        high = min(math.ceil(_yarn_find_dim(self.beta_slow, self.dim, self.base, self.orig)), self.dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(self.dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
        mask = 1.0 - ramp
        return inter * (1 - mask) + extra * mask

    def forward(self, seq_len: int, device, offset: int = 0):
        key = (seq_len, str(device), offset)
        if key not in self._cache:
            pos = torch.arange(seq_len, dtype=torch.float32, device=device) + offset
            cp = state.get_context_parallel_world_size() if state.model_parallel_is_initialized() else 1
            if cp > 1:
                from ..parallel.context_parallel import zigzag_indices
                pos = pos[zigzag_indices(seq_len, cp, state.get_context_parallel_rank(), device)]
            ang = torch.outer(pos, self._inv_freq(device))
            m = yarn_get_mscale(self.factor, self.mscale) / yarn_get_mscale(self.factor, self.mscale_all_dim)
            self._cache = {key: ((ang.cos() * m).contiguous(), (ang.sin() * m).contiguous())}
        return self._cache[key]


class _ReplicatedLinear(nn.Module):
    """y = x W^T with the same weight on every tensor-parallel rank."""

    def __init__(self, config, in_features, out_features, init_method):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=_device(config),
                                               dtype=config.params_dtype))
        if config.perform_initialization:
            init_method(self.weight)
        self.weight.sequence_parallel = config.sequence_parallel     # partial-sum gradient over TP under SP

    def forward(self, x):
        from ..ops.gemm import linear
        return linear(x, self.weight, None)


class MLASelfAttention(nn.Module):
    def __init__(self, config, layer_number: int, causal: bool = True):
        super().__init__()
        from .transformer import Norm
        self.config, self.layer_number, self.causal = config, layer_number, causal
        tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.tp = tp
        self.np = config.num_attention_heads
        self.np_local = self.np // tp
        self.qk_dim, self.pe_dim, self.v_dim = config.qk_head_dim, config.qk_pos_emb_head_dim, config.v_head_dim
        self.q_head = self.qk_dim + self.pe_dim
        self.kv_rank = config.kv_lora_rank
        if config.q_lora_rank is None:
            self.linear_q_proj = ColumnParallelLinear(config.hidden_size, self.np * self.q_head, config=config,
                                                      init_method=config.init_method, bias=False)
        else:
            self.linear_q_down_proj = _ReplicatedLinear(config, config.hidden_size, config.q_lora_rank,
                                                        config.init_method)
            self.q_layernorm = Norm(config, config.q_lora_rank)
            self.linear_q_up_proj = ColumnParallelLinear(config.q_lora_rank, self.np * self.q_head, config=config,
                                                         init_method=config.init_method, bias=False)
        self.linear_kv_down_proj = _ReplicatedLinear(config, config.hidden_size, self.kv_rank + self.pe_dim,
                                                     config.init_method)
        self.kv_layernorm = Norm(config, self.kv_rank)
        self.linear_kv_up_proj = ColumnParallelLinear(self.kv_rank, self.np * (self.qk_dim + self.v_dim),
                                                      config=config, init_method=config.init_method, bias=False)
        self.linear_proj = RowParallelLinear(self.np * self.v_dim, config.hidden_size, config=config,
                                             init_method=config.output_layer_init_method,
                                             bias=config.add_bias_linear, skip_bias_add=True)
        m = yarn_get_mscale(config.rotary_scaling_factor, config.mscale_all_dim) if config.rope_type == "yarn" else 1.0
        self.softmax_scale = m * m / math.sqrt(self.q_head)

    def _qkv(self, x, rotary):
        cfg = self.config
        sp = cfg.sequence_parallel and self.tp > 1
        if cfg.q_lora_rank is None:
            q, _ = self.linear_q_proj(x)
        else:
            q, _ = self.linear_q_up_proj(self.q_layernorm(self.linear_q_down_proj(x)))
        kv = self.linear_kv_down_proj(x)                                      # [s(/tp), b, rank + pe]
        latent, k_pe = kv[..., :self.kv_rank], kv[..., self.kv_rank:]
        kvu, _ = self.linear_kv_up_proj(self.kv_layernorm(latent.contiguous()))
        if sp:
            k_pe = gather_from_sequence_parallel_region(k_pe.contiguous())
        s, b = q.shape[0], q.shape[1]
        q = q.view(s, b, self.np_local, self.q_head)
        kvu = kvu.view(s, b, self.np_local, self.qk_dim + self.v_dim)
        k_pe = k_pe.reshape(s, b, 1, self.pe_dim)
        q_no, q_pe = q[..., :self.qk_dim], q[..., self.qk_dim:]
        k_no, v = kvu[..., :self.qk_dim], kvu[..., self.qk_dim:]
        if rotary is not None:
            cos, sin = rotary
            q_pe = ops.apply_rope(q_pe.contiguous(), cos, sin, cfg.rotary_interleaved)
            k_pe = ops.apply_rope(k_pe.contiguous(), cos, sin, cfg.rotary_interleaved)
        q = torch.cat((q_no, q_pe), dim=-1)
        k = torch.cat((k_no, k_pe.expand(s, b, self.np_local, self.pe_dim)), dim=-1)
        return q, k, v

    def forward(self, hidden_states, rotary=None, inference_context=None, attention_mask=None):
        if inference_context is not None:
            raise NotImplementedError("KV-cache decoding for multi-latent attention is not implemented")
        q, k, v = self._qkv(hidden_states, rotary)
        s, b = q.shape[0], q.shape[1]
        # [s, b, n, d] -> [b, n, s, d]
        o = F.scaled_dot_product_attention(q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3),
                                           is_causal=self.causal, scale=self.softmax_scale,
                                           dropout_p=self.config.attention_dropout if self.training else 0.0)
        o = o.permute(2, 0, 1, 3).reshape(s, b, self.np_local * self.v_dim)
        return self.linear_proj(o)
