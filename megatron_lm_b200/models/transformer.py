"""Transformer building blocks: norm, self/cross attention, MLP, layer, block.

Behavioural parity targets in the reference: ``TransformerLayer``
(megatron/core/transformer/transformer_layer.py:256, forward :432-700),
``TransformerBlock`` (transformer_block.py:258, forward :477-620), ``SelfAttention``
(attention.py:784; fused QKV layout [ng, (np/ng + 2) * hn] :919-965), ``MLP``
(mlp.py:48, forward :127).  There is no spec tree or backend switch: each module
is built directly from the config and calls the sm_100a ops of ``ops/``.
Activations are [s, b, h] throughout.
"""
from __future__ import annotations

import contextlib
import math
from typing import List, Optional

import torch
import torch.nn as nn

from ..config import TransformerConfig
from ..ops import core as ops
from ..ops.attention import attention, fused_qkv_attention
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, _device
from ..parallel.random import CheckpointWithoutOutput, checkpoint, get_cuda_rng_tracker


# --------------------------------------------------------------------------- layer placement
def get_num_layers_to_build(config: TransformerConfig, vp_stage: Optional[int] = None,
                            pp_rank: Optional[int] = None) -> int:
    """Layers held by this (pipeline rank, virtual stage) (reference: transformer_block.py:68)."""
    pp = config.pipeline_model_parallel_size
    if pp_rank is None:
        pp_rank = state.get_pipeline_model_parallel_rank() if state.model_parallel_is_initialized() else 0
    if config.pipeline_model_parallel_layout is not None:
        from .pp_layout import PipelineParallelLayerLayout
        layout = PipelineParallelLayerLayout.from_config(config)
        return layout.get_num_layers_to_build(pp_rank, vp_stage)
    first, last = config.num_layers_in_first_pipeline_stage, config.num_layers_in_last_pipeline_stage
    if first is not None or last is not None:
        middle_ranks = pp - (first is not None) - (last is not None)
        rest = config.num_layers - (first or 0) - (last or 0)
        per_mid = rest // middle_ranks if middle_ranks > 0 else 0
        if pp_rank == 0 and first is not None:
            n = first
        elif pp_rank == pp - 1 and last is not None:
            n = last
        else:
            n = per_mid
    else:
        total = config.num_layers
        if config.account_for_embedding_in_pipeline_split:
            total += 1
        if config.account_for_loss_in_pipeline_split:
            total += 1
        n = total // pp
        if config.account_for_embedding_in_pipeline_split and pp_rank == 0:
            n -= 1
        if config.account_for_loss_in_pipeline_split and pp_rank == pp - 1:
            n -= 1
    vpp = config.virtual_pipeline_model_parallel_size
    if vpp is not None and vpp > 1:
        n //= vpp
    return n


def get_transformer_layer_offset(config: TransformerConfig, vp_stage: Optional[int] = None,
                                 pp_rank: Optional[int] = None) -> int:
    """Global index of this chunk's first layer (reference: transformer_layer.py:37-193).
    With v virtual stages, chunk c of rank r holds layers starting at
    c * (num_layers / v) + r * (num_layers / (pp * v))."""
    pp = config.pipeline_model_parallel_size
    if pp_rank is None:
        pp_rank = state.get_pipeline_model_parallel_rank() if state.model_parallel_is_initialized() else 0
    if pp == 1:
        return 0
    if config.pipeline_model_parallel_layout is not None:
        from .pp_layout import PipelineParallelLayerLayout
        return PipelineParallelLayerLayout.from_config(config).get_layer_offset(pp_rank, vp_stage)
    vpp = config.virtual_pipeline_model_parallel_size or 1
    v = vp_stage or 0
    first, last = config.num_layers_in_first_pipeline_stage, config.num_layers_in_last_pipeline_stage
    if first is not None or last is not None:
        middle_ranks = pp - (first is not None) - (last is not None)
        rest = config.num_layers - (first or 0) - (last or 0)
        per_mid = rest // middle_ranks if middle_ranks > 0 else 0
        sizes = [(first if (r == 0 and first is not None) else last if (r == pp - 1 and last is not None) else per_mid)
                 for r in range(pp)]
        per_chunk = [s // vpp for s in sizes]
        return v * sum(per_chunk) + sum(per_chunk[:pp_rank])
    total = config.num_layers + int(config.account_for_embedding_in_pipeline_split) + \
        int(config.account_for_loss_in_pipeline_split)
    per_rank = total // pp
    per_chunk = per_rank // vpp
    off = v * (total // vpp) + pp_rank * per_chunk
    if config.account_for_embedding_in_pipeline_split and not (pp_rank == 0 and v == 0):
        off -= 1
    return off


# --------------------------------------------------------------------------- norm
class Norm(nn.Module):
    """LayerNorm or RMSNorm over the last dim with the fused fwd/bwd kernels."""

    def __init__(self, config: TransformerConfig, hidden_size: int, eps: Optional[float] = None):
        super().__init__()
        self.rms = config.normalization == "RMSNorm"
        if config.normalization not in ("LayerNorm", "RMSNorm"):
            raise ValueError(f"unknown normalization {config.normalization}")
        self.eps = config.layernorm_epsilon if eps is None else eps
        self.zero_centered = config.layernorm_zero_centered_gamma
        dev = _device(config)
        init = torch.zeros if self.zero_centered else torch.ones
        self.weight = nn.Parameter(init(hidden_size, device=dev, dtype=config.params_dtype))
        if not self.rms:
            self.bias = nn.Parameter(torch.zeros(hidden_size, device=dev, dtype=config.params_dtype))
        else:
            self.register_parameter("bias", None)
        # gradients of these replicated parameters are partial sums under sequence parallelism
        for p in self.parameters():
            p.sequence_parallel = config.sequence_parallel

    def forward(self, x):
        if self.rms:
            return ops.rmsnorm(x, self.weight, self.eps, self.zero_centered)
        return ops.layernorm(x, self.weight, self.bias, self.eps, self.zero_centered)


class L2Norm(nn.Module):
    """x / sqrt(mean(x^2) + eps) over the last dim, no parameters (reference: transformer/torch_norm.py:54);
    the q/k normalisation of ``qk_l2_norm`` models."""

    def __init__(self, hidden_size: int = 0, eps: float = 1e-6, **_):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x)


class WrappedTorchNorm(nn.Module):
    """The plain-PyTorch norm of the reference's local spec (transformer/torch_norm.py:9), for configurations the
    fused kernels do not cover (hidden size not a multiple of 8) and as their numerical reference."""

    def __init__(self, config: TransformerConfig, hidden_size: int, eps: float = 1e-5, **_):
        super().__init__()
        if config.layernorm_zero_centered_gamma:
            raise ValueError("zero-centred gamma needs the fused norm")
        if config.normalization == "LayerNorm":
            self.norm = nn.LayerNorm(hidden_size, eps=eps)
        elif config.normalization == "RMSNorm":
            self.norm = nn.RMSNorm(hidden_size, eps=eps)
        else:
            raise ValueError(f"unknown normalization {config.normalization}")
        for p in self.norm.parameters():
            p.sequence_parallel = config.sequence_parallel

    def forward(self, x):
        return self.norm(x)


class IdentityOp(nn.Module):
    """Returns its first argument (reference: transformer/identity_op.py:5): the placeholder a layer spec uses for
    a sub-module it leaves out."""

    def __init__(self, *a, **k):
        super().__init__()

    def forward(self, x, *a, **k):
        return x


class IdentityFuncOp(IdentityOp):
    """Returns a function that returns its argument (the bias-dropout-add slot of a spec)."""

    def forward(self, *a, **k):
        return super().forward


# --------------------------------------------------------------------------- attention
def _rope_copy(qkv5, cos, sin, interleaved):
    """Out-of-place RoPE on q and k of a fused QKV tensor (inference path, no autograd)."""
    out = qkv5.clone()
    view = out[:, :, :, :-1]
    ops._rope_launch(view, view, cos, sin, interleaved, 1.0)
    return out


def masked_attention(q5, k, v, attention_mask, scale, causal=False, window=None):
    """Attention with an arbitrary mask (True = may not attend), e.g. padding masks of BERT / T5 batches.
    q5 [sq, b, ng, qpg, d], k/v [sk, b, ng, d], mask broadcastable to [b, 1, sq, sk].  The flash kernels
    cover the causal and full cases; arbitrary masks go through torch's scaled-dot-product attention."""
    sq, b, ng, qpg, d = q5.shape
    sk = k.shape[0]
    q = q5.reshape(sq, b, ng * qpg, d).permute(1, 2, 0, 3)
    kk = k.permute(1, 2, 0, 3).repeat_interleave(qpg, dim=1)
    vv = v.permute(1, 2, 0, 3).repeat_interleave(qpg, dim=1)
    allow = ~attention_mask.bool()
    if causal:
        allow = allow & torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(sk - sq)
        if window is not None:
            allow = allow & torch.ones(sq, sk, dtype=torch.bool, device=q.device).triu(sk - sq - window)
    o = torch.nn.functional.scaled_dot_product_attention(q, kk, vv, attn_mask=allow, scale=scale)
    return o.permute(2, 0, 1, 3).reshape(sq, b, ng * qpg * d)


class SelfAttention(nn.Module):
    def __init__(self, config: TransformerConfig, layer_number: int, causal: bool = True):
        super().__init__()
        self.config, self.layer_number, self.causal = config, layer_number, causal
        tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.hn = config.kv_channels
        self.np, self.ng = config.num_attention_heads, config.num_query_groups
        if self.ng % tp != 0:
            raise ValueError("num_query_groups must be divisible by the tensor-parallel size")
        self.np_local, self.ng_local = self.np // tp, self.ng // tp
        self.qpg = self.np // self.ng
        qkv_out = (self.np + 2 * self.ng) * self.hn
        self.linear_qkv = ColumnParallelLinear(config.hidden_size, qkv_out, config=config,
                                               init_method=config.init_method,
                                               bias=config.add_bias_linear or config.add_qkv_bias)
        self.linear_proj = RowParallelLinear(self.np * self.hn, config.hidden_size, config=config,
                                             init_method=config.output_layer_init_method,
                                             bias=config.add_bias_linear, skip_bias_add=True)
        if getattr(config, "qk_l2_norm", False):
            self.q_layernorm, self.k_layernorm = L2Norm(self.hn), L2Norm(self.hn)
        elif config.qk_layernorm:
            self.q_layernorm = Norm(config, self.hn)
            self.k_layernorm = Norm(config, self.hn)
        else:
            self.q_layernorm = self.k_layernorm = None
        scale = config.softmax_scale if config.softmax_scale is not None else 1.0 / math.sqrt(self.hn)
        self.softmax_scale = scale
        # sliding window: window_size = (left, 0) on a causal layer - a query sees itself and `left` keys before it
        self.window = None
        if config.window_size is not None:
            left, right = config.window_size
            if not causal or right not in (0, -1) or left < 0:
                raise NotImplementedError("window_size is implemented as the causal window (left, 0)")
            self.window = int(left)
        self.recompute_core = config.recompute_granularity == "selective" and "core_attn" in config.recompute_modules
        # layers without rotary embedding: every no_rope_freq-th layer, or an explicit 0 / 1 list (1 = no rotary)
        nrf = getattr(config, "no_rope_freq", None)
        if isinstance(nrf, int) and nrf > 0:
            self.no_rope = layer_number % nrf == 0
        elif isinstance(nrf, (list, tuple)):
            self.no_rope = bool(nrf[(layer_number - 1) % len(nrf)])
        else:
            self.no_rope = False
        self.cp_size = state.get_context_parallel_world_size() if state.model_parallel_is_initialized() else 1
        ct = config.cp_comm_type
        self.cp_comm_type = (ct[(layer_number - 1) % len(ct)] if isinstance(ct, (list, tuple)) else ct) or "p2p"

    def _core(self, qkv5, cos=None, sin=None):
        rope = None if cos is None else (cos, sin)
        return fused_qkv_attention(qkv5, causal=self.causal, scale=self.softmax_scale, rope=rope,
                                   rotary_interleaved=self.config.rotary_interleaved, window=self.window)

    def forward(self, hidden_states, rotary=None, inference_context=None, attention_mask=None):
        qkv, _ = self.linear_qkv(hidden_states)                       # [s, b, (np+2ng)/tp * hn]
        s, b = qkv.shape[0], qkv.shape[1]
        qkv5 = qkv.view(s, b, self.ng_local, self.qpg + 2, self.hn)
        if self.q_layernorm is not None:
            q = self.q_layernorm(qkv5[:, :, :, :self.qpg].contiguous())
            k = self.k_layernorm(qkv5[:, :, :, self.qpg:self.qpg + 1].contiguous())
            qkv5 = torch.cat((q, k, qkv5[:, :, :, self.qpg + 1:]), dim=3)
        cos, sin = rotary if rotary is not None and not self.no_rope else (None, None)
        if self.window is not None and (inference_context is not None or self.cp_size > 1):
            raise NotImplementedError("sliding-window attention is not available with context parallelism or the "
                                      "inference engines' key/value caches")
        if self.cp_size > 1 and inference_context is None:
            # context parallel: q/k/v leave the fused buffer (K/V travel between ranks)
            from ..parallel.context_parallel import context_parallel_attention
            q = qkv5[:, :, :, :self.qpg].reshape(s, b, self.ng_local * self.qpg, self.hn)
            k = qkv5[:, :, :, self.qpg]
            v = qkv5[:, :, :, self.qpg + 1]
            if cos is not None:
                q = ops.apply_rope(q, cos, sin, self.config.rotary_interleaved)
                k = ops.apply_rope(k, cos, sin, self.config.rotary_interleaved)
            ctx_out = context_parallel_attention(q.reshape(s, b, self.ng_local, self.qpg, self.hn), k.contiguous(),
                                                 v.contiguous(), self.cp_comm_type, scale=self.softmax_scale,
                                                 causal=self.causal)
            out, bias = self.linear_proj(ctx_out.reshape(s, b, self.np_local * self.hn))
            return out, bias
        from ..packed_seq_params import PackedSegments
        if isinstance(attention_mask, PackedSegments) and inference_context is None:
            # packed row: every document is its own causal attention problem on a slice of the fused buffer
            # (sequence parallelism has already gathered the row: qkv5 holds all tokens of this rank's heads)
            outs = []
            bnd = attention_mask.bounds
            for s0, s1 in zip(bnd[:-1], bnd[1:]):
                if s1 > s0:
                    outs.append(self._core(qkv5[s0:s1], None if cos is None else cos[s0:s1],
                                           None if sin is None else sin[s0:s1]))
            ctx_out = outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)
        elif attention_mask is not None and inference_context is None:
            if cos is not None:
                qkv5 = ops.apply_rope_qkv_(qkv5.clone() if qkv5.is_cuda else qkv5, cos, sin,
                                           self.config.rotary_interleaved)
            ctx_out = masked_attention(qkv5[:, :, :, :self.qpg], qkv5[:, :, :, self.qpg], qkv5[:, :, :, self.qpg + 1],
                                       attention_mask, self.softmax_scale, self.causal, self.window)
        elif inference_context is not None:
            if cos is not None:
                qkv5 = _rope_copy(qkv5, cos, sin, self.config.rotary_interleaved) if qkv5.is_cuda else \
                    ops.apply_rope_qkv_(qkv5, cos, sin, self.config.rotary_interleaved)
            ctx_out = inference_context.attend(self.layer_number, qkv5, self.softmax_scale)
        elif self.recompute_core and self.training:
            # the in-place rotation must not run twice on one buffer: recompute works on a copy
            ctx_out = checkpoint(lambda t, c, s_: self._core(t.clone() if t.is_cuda else t, c, s_), False,
                                 qkv5, cos, sin)
        else:
            ctx_out = self._core(qkv5, cos, sin)                      # [s, b, np_local * hn]
        out, bias = self.linear_proj(ctx_out)
        return out, bias


class CrossAttention(nn.Module):
    """Queries from the decoder stream, keys/values from an encoder output
    (reference: attention.py:981)."""

    def __init__(self, config: TransformerConfig, layer_number: int):
        super().__init__()
        self.config = config
        tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.hn, self.np = config.kv_channels, config.num_attention_heads
        self.np_local = self.np // tp
        self.linear_q = ColumnParallelLinear(config.hidden_size, self.np * self.hn, config=config,
                                             init_method=config.init_method, bias=config.add_bias_linear)
        self.linear_kv = ColumnParallelLinear(config.hidden_size, 2 * self.np * self.hn, config=config,
                                              init_method=config.init_method, bias=config.add_bias_linear)
        self.linear_proj = RowParallelLinear(self.np * self.hn, config.hidden_size, config=config,
                                             init_method=config.output_layer_init_method,
                                             bias=config.add_bias_linear, skip_bias_add=True)

    def forward(self, hidden_states, key_value_states, attention_mask=None):
        q, _ = self.linear_q(hidden_states)
        kv, _ = self.linear_kv(key_value_states)
        sq, b = q.shape[0], q.shape[1]
        sk = kv.shape[0]
        q5 = q.view(sq, b, self.np_local, 1, self.hn)
        kv5 = kv.view(sk, b, self.np_local, 2, self.hn)
        if attention_mask is not None:
            o = masked_attention(q5, kv5[:, :, :, 0], kv5[:, :, :, 1], attention_mask, 1.0 / math.sqrt(self.hn))
        else:
            o = attention(q5, kv5[:, :, :, 0], kv5[:, :, :, 1], causal=False)
        return self.linear_proj(o.reshape(sq, b, self.np_local * self.hn))


# --------------------------------------------------------------------------- MLP
class MLP(nn.Module):
    def __init__(self, config: TransformerConfig, ffn_hidden_size: Optional[int] = None, is_expert: bool = False):
        super().__init__()
        self.config = config
        ffn = ffn_hidden_size or config.ffn_hidden_size
        self.gated = config.gated_linear_unit
        act = config.activation_func if isinstance(config.activation_func, str) else getattr(
            config.activation_func, "__name__", "gelu")
        self.act = {"silu": "silu", "swiglu": "silu", "gelu": "gelu", "relu": "relu",
                    "squared_relu": "squared_relu"}.get(act, act)
        from ..activations import BY_NAME
        # anything else: a named elementwise function, or the callable itself
        self.act_fn = BY_NAME.get(self.act) or (config.activation_func if callable(config.activation_func) else None)
        if self.act_fn is None:
            raise ValueError(f"unsupported activation {act}")
        self.linear_fc1 = ColumnParallelLinear(config.hidden_size, ffn * (2 if self.gated else 1), config=config,
                                               init_method=config.init_method, bias=config.add_bias_linear,
                                               skip_bias_add=True, is_expert=is_expert,
                                               stride=2 if self.gated else 1)
        self.linear_fc2 = RowParallelLinear(ffn, config.hidden_size, config=config,
                                            init_method=config.output_layer_init_method,
                                            bias=config.add_bias_linear, skip_bias_add=True, is_expert=is_expert)

    def activation(self, x, bias):
        if self.gated:
            if bias is not None:
                x = x + bias
            if self.act == "silu":
                return ops.swiglu(x)
            a, b = x.chunk(2, dim=-1)
            return self.act_fn(a) * b
        if self.act == "gelu":
            return ops.bias_gelu(x, bias)
        if bias is not None:
            x = x + bias
        if self.act == "relu":
            return torch.relu(x)
        if self.act == "squared_relu":
            return torch.relu(x).pow(2)
        return self.act_fn(x)

    def forward(self, hidden_states):
        h, b1 = self.linear_fc1(hidden_states)
        h = self.activation(h, b1)
        return self.linear_fc2(h)


# --------------------------------------------------------------------------- layer / block
def _build_slot(spec, **pool):
    """Instantiate the class a layer spec names for one slot.  The class receives those of ``pool`` (config,
    layer_number, hidden_size, causal) that its constructor names, plus the spec's own ``params`` where the
    constructor accepts them; identity placeholders take nothing."""
    import inspect
    from .spec_utils import ModuleSpec, get_module
    cls = get_module(spec) if isinstance(spec, ModuleSpec) else spec
    params = dict(spec.params) if isinstance(spec, ModuleSpec) else {}
    if isinstance(cls, type) and issubclass(cls, IdentityOp):
        return cls()
    sig = inspect.signature(cls.__init__ if isinstance(cls, type) else cls)
    names = set(sig.parameters)
    takes_kw = any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values())
    kw = {k: v for k, v in pool.items() if k in names}
    kw.update({k: v for k, v in params.items() if k in names or takes_kw})
    return cls(**kw)


class TransformerLayer(nn.Module):
    """Pre-norm residual block: x + drop(attn(norm(x)) + b); x + drop(mlp(norm(x)) + b)."""

    def __init__(self, config: TransformerConfig, layer_number: int, is_moe: bool = False, causal: bool = True,
                 cross_attention: bool = False, submodules=None):
        """``submodules`` (a ``TransformerLayerSubmodules``) names the class of each slot; slots it leaves empty,
        and all slots without it, take this library's modules as the config describes them."""
        super().__init__()
        self.config, self.layer_number = config, layer_number
        sub = submodules

        def slot(name, default):
            spec = getattr(sub, name, None) if sub is not None else None
            if spec is None or isinstance(spec, str):
                return default()
            return _build_slot(spec, config=config, layer_number=layer_number, hidden_size=config.hidden_size,
                               causal=causal)

        def default_attention():
            if getattr(config, "multi_latent_attention", False):
                from .mla import MLASelfAttention
                return MLASelfAttention(config, layer_number, causal=causal)
            return SelfAttention(config, layer_number, causal=causal)

        def default_mlp():
            if is_moe:
                from .moe import MoELayer
                return MoELayer(config, layer_number)
            return MLP(config)

        self.input_layernorm = slot("input_layernorm", lambda: Norm(config, config.hidden_size))
        self.self_attention = slot("self_attention", default_attention)
        if cross_attention:
            self.pre_cross_attn_layernorm = slot("pre_cross_attn_layernorm", lambda: Norm(config, config.hidden_size))
            self.cross_attention = slot("cross_attention", lambda: CrossAttention(config, layer_number))
        else:
            self.cross_attention = None
        self.pre_mlp_layernorm = slot("pre_mlp_layernorm", lambda: Norm(config, config.hidden_size))
        self.mlp = slot("mlp", default_mlp)
        from .moe import MoELayer as _MoE
        self.is_moe = isinstance(self.mlp, _MoE)
        self.hidden_dropout = config.hidden_dropout
        mods = config.recompute_modules if config.recompute_granularity == "selective" else []
        self.post_ln_residual = config.apply_residual_connection_post_layernorm
        self.recompute_input_ln = "layernorm" in mods and not self.post_ln_residual
        self.recompute_mlp = "mlp" in mods or (self.is_moe and ("moe" in mods or config.moe_layer_recompute))
        if config.fp8:
            from ..fp8_utils import mark_layer_precision
            mark_layer_precision(self, config, layer_number - 1)       # first / last layers may stay in 16 bits
        if getattr(config, "delay_wgrad_compute", False):
            # the weight-gradient GEMMs of this layer's linears are queued by backward and run by backward_dw():
            # the expert-parallel overlap schedule places them under the other micro-batch's communication
            # (reference: transformer_layer.py backward_dw, attention.py:~970, --delay-wgrad-compute)
            from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
            for m in self.modules():
                if isinstance(m, (ColumnParallelLinear, RowParallelLinear)) and m.weight is not None:
                    m.weight.defer_wgrad = True

    def backward_dw(self) -> int:
        """Run the queued weight-gradient products of this layer's linears; returns how many ran."""
        from ..parallel.layers import drain_deferred_wgrads
        return drain_deferred_wgrads(only={id(p) for p in self.parameters()})

    def _bda(self, x, bias, residual):
        p = self.hidden_dropout
        if p > 0.0 and self.training and self.config.sequence_parallel:
            with get_cuda_rng_tracker().fork():
                seed = int(torch.randint(0, 2 ** 31 - 1, (1,)).item()) if not x.is_cuda else None
                return ops.bias_dropout_add(x, bias, residual, p, True, seed)
        return ops.bias_dropout_add(x, bias, residual, p, self.training)

    def forward(self, hidden_states, rotary=None, inference_context=None, encoder_output=None,
                attention_mask=None, enc_dec_attn_mask=None):
        residual = hidden_states
        if self.recompute_input_ln and self.training:
            ck = CheckpointWithoutOutput()
            ln = ck.checkpoint(self.input_layernorm, hidden_states)
        else:
            ck, ln = None, self.input_layernorm(hidden_states)
        if self.post_ln_residual:
            residual = ln                         # the residual branch starts after the norm
        attn_out, attn_bias = self.self_attention(ln, rotary=rotary, inference_context=inference_context,
                                                  attention_mask=attention_mask)
        if ck is not None:
            ck.discard_output_and_register_recompute(attn_out)
        hidden_states = self._bda(attn_out, attn_bias, residual)
        if self.cross_attention is not None:
            residual = hidden_states
            ln = self.pre_cross_attn_layernorm(hidden_states)
            x_out, x_bias = self.cross_attention(ln, encoder_output, enc_dec_attn_mask)
            hidden_states = self._bda(x_out, x_bias, residual)
        residual = hidden_states
        if self.recompute_input_ln and self.training and not self.is_moe:
            ck = CheckpointWithoutOutput()
            ln = ck.checkpoint(self.pre_mlp_layernorm, hidden_states)
        else:
            ck, ln = None, self.pre_mlp_layernorm(hidden_states)
        if self.post_ln_residual:
            residual = ln
        if self.recompute_mlp and self.training:
            mlp_out, mlp_bias = checkpoint(self.mlp, False, ln)
        else:
            mlp_out, mlp_bias = self.mlp(ln)
        if ck is not None:
            ck.discard_output_and_register_recompute(mlp_out)
        return self._bda(mlp_out, mlp_bias, residual)


class TransformerBlock(nn.Module):
    """The layers of one pipeline (virtual) stage, plus the final norm on the last stage."""

    def __init__(self, config: TransformerConfig, pre_process: bool = True, post_process: bool = True,
                 vp_stage: Optional[int] = None, causal: bool = True, cross_attention: bool = False,
                 post_layer_norm: bool = True, spec=None):
        """``spec``: None, one layer ``ModuleSpec`` (used for every layer) or a ``TransformerBlockSubmodules`` whose
        ``layer_specs`` list covers the whole model (this stage takes its slice) or just this stage."""
        super().__init__()
        from .gpt_layer_specs import TransformerBlockSubmodules, layer_spec_is_moe
        from .spec_utils import ModuleSpec, get_module
        self.config, self.pre_process, self.post_process, self.vp_stage = config, pre_process, post_process, vp_stage
        n = get_num_layers_to_build(config, vp_stage)
        self.layer_offset = get_transformer_layer_offset(config, vp_stage)
        pattern = config.moe_layer_pattern()

        def layer_spec(i):
            if spec is None:
                return None
            if isinstance(spec, TransformerBlockSubmodules):
                specs = spec.layer_specs or []
                if len(specs) == n:
                    return specs[i]
                if len(specs) == config.num_layers:
                    return specs[self.layer_offset + i]
                raise ValueError(f"block spec lists {len(specs)} layers; the stage builds {n} of {config.num_layers}")
            if isinstance(spec, ModuleSpec):
                return spec
            raise TypeError(f"unsupported transformer layer spec {type(spec).__name__}")

        layers = []
        hetero = getattr(config, "heterogeneous_layers_config_encoded_json", None)
        if hetero:
            # every layer from its own block configuration (attention / MLP absent, linear, or of another width)
            from .heterogeneous import build_heterogeneous_layers
            if not causal or cross_attention:
                raise NotImplementedError("heterogeneous layer configurations are for decoder-only models")
            layers = list(build_heterogeneous_layers(config, hetero, offset=self.layer_offset, count=n))
            n = 0
        for i in range(n):
            ls = layer_spec(i)
            cls = get_module(ls) if ls is not None else TransformerLayer
            moe = layer_spec_is_moe(ls)
            kw = dict(is_moe=bool(pattern[self.layer_offset + i]) if moe is None else moe, causal=causal,
                      cross_attention=cross_attention)
            if ls is not None and ls.submodules is not None:
                kw["submodules"] = ls.submodules
            layers.append(cls(config, self.layer_offset + i + 1, **kw))
        self.layers = nn.ModuleList(layers)
        norm_cls = getattr(spec, "layer_norm", None) if isinstance(spec, TransformerBlockSubmodules) else None
        if post_process and post_layer_norm:
            self.final_layernorm = _build_slot(norm_cls, config=config, hidden_size=config.hidden_size) \
                if norm_cls is not None else Norm(config, config.hidden_size)
        else:
            self.final_layernorm = None
        self.input_tensor = None

    def set_input_tensor(self, t):
        """Activations received from the previous pipeline stage replace the forward input."""
        self.input_tensor = t

    def _run_layers(self, start, end):
        def fn(h, cos, sin):
            rotary = None if cos is None else (cos, sin)
            for i in range(start, end):
                h = self.layers[i](h, rotary=rotary)
            return h
        return fn

    def forward(self, hidden_states, rotary=None, inference_context=None, encoder_output=None,
                attention_mask=None, enc_dec_attn_mask=None):
        if not self.pre_process and self.input_tensor is not None:
            hidden_states = self.input_tensor
        cfg = self.config
        full = cfg.recompute_granularity == "full" and self.training
        cos, sin = (None, None) if rotary is None else rotary
        if full:
            n = len(self.layers)
            if cfg.recompute_method == "uniform":
                step = cfg.recompute_num_layers
                i = 0
                while i < n:
                    hidden_states = checkpoint(self._run_layers(i, min(i + step, n)), False, hidden_states, cos, sin)
                    i += step
            else:   # block: recompute only the first recompute_num_layers layers
                for i in range(n):
                    if i < cfg.recompute_num_layers:
                        hidden_states = checkpoint(self._run_layers(i, i + 1), False, hidden_states, cos, sin)
                    else:
                        hidden_states = self.layers[i](hidden_states, rotary=rotary)
        else:
            # cpu_offloading: what the first cpu_offloading_num_layers layers keep for backward lives in (pinned) host
            # memory between the passes and comes back when backward reaches the layer
            # (reference: megatron/core/extensions/transformer_engine.py get_cpu_offload_context)
            n_off = cfg.cpu_offloading_num_layers if (cfg.cpu_offloading and self.training
                                                      and torch.is_grad_enabled()) else 0
            for i, layer in enumerate(self.layers):
                ctx = torch.autograd.graph.save_on_cpu(pin_memory=hidden_states.is_cuda) if i < n_off \
                    else contextlib.nullcontext()
                with ctx:
                    hidden_states = layer(hidden_states, rotary=rotary, inference_context=inference_context,
                                          encoder_output=encoder_output, attention_mask=attention_mask,
                                          enc_dec_attn_mask=enc_dec_attn_mask)
        if self.final_layernorm is not None:
            hidden_states = self.final_layernorm(hidden_states)
        return hidden_states
