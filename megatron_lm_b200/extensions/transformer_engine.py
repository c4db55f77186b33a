"""The module names of the reference's Transformer Engine adapter
(megatron/core/extensions/transformer_engine.py: TENorm :79, TELinear :116, TELayerNormColumnParallelLinear :328,
TEColumnParallelLinear :518, TERowParallelLinear :611, TEDotProductAttention :705, TEGroupedLinear :864,
TEDelayedScaling :1196, te_checkpoint :1297, get_cpu_offload_context :1346), implemented on this library's own
sm_100a kernels.  Nothing here wraps an external library: each class is the native module that does the same job
(the fused norm / GEMM / attention kernels of ``ops/``), under the name and call contract the reference's layer
specs use - linear layers return ``(output, bias_or_None)``, attention takes [s, b, heads, d] tensors.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..config import TransformerConfig
from ..ops import attention as attn_ops
from ..ops.fp8 import DelayedScalingState
from ..ops.grouped_gemm import grouped_linear
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, _device
from ..parallel.random import CudaRNGStatesTracker as _CudaRNGStatesTracker
from ..parallel.random import checkpoint as _checkpoint
from ..models.transformer import MLP as _MLP
from ..models.transformer import Norm, masked_attention

HAVE_TE = False          # no external library is used; kept because callers of the reference test this name


class TENorm:
    """Factory with the reference's call shape ``TENorm(config, hidden_size, eps)`` returning the fused norm."""

    def __new__(cls, config: TransformerConfig, hidden_size: int, eps: float = 1e-5):
        return Norm(config, hidden_size, eps)


class TEColumnParallelLinear(ColumnParallelLinear):
    def __init__(self, input_size, output_size, *, config, init_method, gather_output=False, bias=True,
                 skip_bias_add=False, is_expert=False, skip_weight_param_allocation=False, tp_comm_buffer_name=None,
                 tp_group=None, **_):
        super().__init__(input_size, output_size, config=config, init_method=init_method, bias=bias,
                         gather_output=gather_output, skip_bias_add=skip_bias_add, is_expert=is_expert,
                         tp_group=tp_group, skip_weight_param_allocation=skip_weight_param_allocation)


class TERowParallelLinear(RowParallelLinear):
    def __init__(self, input_size, output_size, *, config, init_method, bias=True, input_is_parallel=True,
                 skip_bias_add=False, is_expert=False, tp_comm_buffer_name=None, tp_group=None, **_):
        super().__init__(input_size, output_size, config=config, init_method=init_method, bias=bias,
                         input_is_parallel=input_is_parallel, skip_bias_add=skip_bias_add, is_expert=is_expert,
                         tp_group=tp_group)


class TELinear(nn.Module):
    """``parallel_mode`` in {"column", "row", "duplicated", None} selects the sharding, as in the reference."""

    def __init__(self, input_size, output_size, *, parallel_mode: Optional[str], config, init_method, bias=True,
                 skip_bias_add=False, skip_weight_param_allocation=False, tp_comm_buffer_name=None, is_expert=False,
                 **_):
        super().__init__()
        self.parallel_mode = parallel_mode
        if parallel_mode == "column":
            self.inner = ColumnParallelLinear(input_size, output_size, config=config, init_method=init_method,
                                              bias=bias, skip_bias_add=skip_bias_add, is_expert=is_expert)
        elif parallel_mode == "row":
            self.inner = RowParallelLinear(input_size, output_size, config=config, init_method=init_method, bias=bias,
                                           skip_bias_add=skip_bias_add, is_expert=is_expert)
        elif parallel_mode in (None, "duplicated"):
            self.inner = nn.Linear(input_size, output_size, bias=bias, device=_device(config),
                                   dtype=config.params_dtype)
            with torch.no_grad():
                init_method(self.inner.weight)
                if bias:
                    self.inner.bias.zero_()
            self.skip_bias_add = skip_bias_add
        else:
            raise ValueError(f"unknown parallel mode {parallel_mode}")

    def forward(self, x):
        if isinstance(self.inner, nn.Linear):
            if self.skip_bias_add and self.inner.bias is not None:
                return torch.nn.functional.linear(x, self.inner.weight), self.inner.bias
            return self.inner(x), None
        return self.inner(x)


class TELayerNormColumnParallelLinear(nn.Module):
    """Norm followed by a column-parallel linear layer, one module (parameter names ``layer_norm_weight`` /
    ``layer_norm_bias`` / ``weight`` / ``bias`` as in the reference's checkpoints)."""

    def __init__(self, input_size, output_size, *, config, init_method, gather_output=False, bias=True,
                 skip_bias_add=False, is_expert=False, skip_weight_param_allocation=False, tp_comm_buffer_name=None,
                 tp_group=None, **_):
        super().__init__()
        norm = Norm(config, input_size)
        self.rms, self.eps, self.zero_centered = norm.rms, norm.eps, norm.zero_centered
        self.layer_norm_weight = norm.weight
        self.layer_norm_bias = norm.bias
        self.linear = ColumnParallelLinear(input_size, output_size, config=config, init_method=init_method, bias=bias,
                                           gather_output=gather_output, skip_bias_add=skip_bias_add,
                                           is_expert=is_expert, tp_group=tp_group)

    @property
    def weight(self):
        return self.linear.weight

    @property
    def bias(self):
        return self.linear.bias

    def forward(self, x):
        from ..ops import core as ops
        if self.rms:
            h = ops.rmsnorm(x, self.layer_norm_weight, self.eps, self.zero_centered)
        else:
            h = ops.layernorm(x, self.layer_norm_weight, self.layer_norm_bias, self.eps, self.zero_centered)
        return self.linear(h)


class TEDotProductAttention(nn.Module):
    """Core attention on [s, b, heads, d] query and [s, b, groups, d] key / value tensors; returns [s, b, heads*d].
    Causal and full attention run the flash kernels; an explicit mask goes through the masked path."""

    def __init__(self, config: TransformerConfig, layer_number: int = 1, attn_mask_type="causal",
                 attention_type: str = "self", attention_dropout: Optional[float] = None,
                 softmax_scale: Optional[float] = None, k_channels: Optional[int] = None,
                 v_channels: Optional[int] = None, cp_comm_type: str = "p2p", model_comm_pgs=None, **_):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        name = getattr(attn_mask_type, "name", attn_mask_type)
        self.causal = name in ("causal", "padding_causal")
        d = k_channels or config.kv_channels
        self.scale = softmax_scale if softmax_scale is not None else d ** -0.5

    def forward(self, query, key, value, attention_mask=None, attn_mask_type=None, attention_bias=None,
                packed_seq_params=None):
        if attn_mask_type is not None:
            name = getattr(attn_mask_type, "name", attn_mask_type)
            causal = name in ("causal", "padding_causal")
        else:
            causal = self.causal
        sq, b, nh, d = query.shape
        ng = key.shape[2]
        q5 = query.reshape(sq, b, ng, nh // ng, d)
        if attention_mask is not None:
            o = masked_attention(q5, key, value, attention_mask, self.scale, causal=causal)
        else:
            o = attn_ops.attention(q5, key, value, causal=causal, scale=self.scale)
        return o.reshape(sq, b, nh * d)


class TEGroupedLinear(nn.Module):
    """``num_gemms`` independent linear layers applied to consecutive row groups of the input
    (``forward(x, m_splits)``), one ragged grouped GEMM launch."""

    def __init__(self, num_gemms: int, input_size: int, output_size: int, *, parallel_mode: Optional[str], config,
                 init_method, bias: bool = False, skip_bias_add: bool = False, is_expert: bool = True,
                 tp_comm_buffer_name=None, **_):
        super().__init__()
        if bias:
            raise ValueError("grouped expert layers carry no bias")
        etp = state.get_expert_tensor_parallel_world_size() if state.model_parallel_is_initialized() else 1
        out_l, in_l = output_size, input_size
        if parallel_mode == "column":
            out_l //= etp
        elif parallel_mode == "row":
            in_l //= etp
        self.weight = nn.Parameter(torch.empty(num_gemms, out_l, in_l, device=_device(config),
                                               dtype=config.params_dtype))
        with torch.no_grad():
            for e in range(num_gemms):
                init_method(self.weight[e])
        self.weight.allreduce = not (config.expert_model_parallel_size > 1)

    def forward(self, x, m_splits):
        return grouped_linear(x, self.weight, m_splits), None


class TEColumnParallelGroupedLinear(TEGroupedLinear):
    def __init__(self, num_gemms, input_size, output_size, **kw):
        kw.pop("parallel_mode", None)
        super().__init__(num_gemms, input_size, output_size, parallel_mode="column", **kw)


class TERowParallelGroupedLinear(TEGroupedLinear):
    def __init__(self, num_gemms, input_size, output_size, **kw):
        kw.pop("parallel_mode", None)
        super().__init__(num_gemms, input_size, output_size, parallel_mode="row", **kw)


class TEDelayedScaling(DelayedScalingState):
    """FP8 delayed-scaling recipe state (amax history -> scale), under the reference's name."""

    def __init__(self, config: Optional[TransformerConfig] = None, fp8_format: str = "hybrid", margin: int = 0,
                 device="cpu", **kw):
        hist = kw.pop("amax_history_len", getattr(config, "fp8_amax_history_len", 1) if config is not None else 1)
        algo = kw.pop("amax_compute_algo", getattr(config, "fp8_amax_compute_algo", "most_recent")
                      if config is not None else "most_recent")
        super().__init__(fmt=0, history_len=hist, algo=algo, margin=margin, device=device)
        self.fp8_format = fp8_format


def te_checkpoint(forward_func, distribute_saved_activations, get_rng_state_tracker, tp_group, *args, **kwargs):
    """Activation recomputation with RNG replay (the reference forwards this to the external library)."""
    return _checkpoint(forward_func, distribute_saved_activations, *args)


def get_cpu_offload_context(enabled, num_layers, model_layers, activation_offloading, weight_offloading):
    """(context manager, sync function) for activation offloading to host memory: saved tensors of the wrapped
    region move to pinned host memory on pack and come back on unpack."""
    import contextlib
    if not enabled:
        return contextlib.nullcontext(), (lambda t: t)
    ctx = torch.autograd.graph.save_on_cpu(pin_memory=torch.cuda.is_available())
    return ctx, (lambda t: t)


class TEFusedMLP(_MLP):
    """The MLP with norm, bias, activation and both projections as fused kernels - which the native MLP already is
    (fused norm + GEMM epilogues + SwiGLU kernel), so the class only carries the adapter's name
    (reference: transformer_engine.py:1353 ``TEFusedMLP`` built from the library's fusible ops)."""


class TECudaRNGStatesTracker(_CudaRNGStatesTracker):
    """The adapter's name for the RNG-state tracker (reference: transformer_engine.py:1498)."""

    def is_initialized(self) -> bool:
        return bool(getattr(self, "states_", None))


def SplitAlongDim(tensor: torch.Tensor, dim: int, split_sizes):
    """Views of ``tensor`` cut along ``dim`` (reference: the library's ``_SplitAlongDim.apply``; autograd handles the
    concatenation of the gradients)."""
    return torch.split(tensor, list(split_sizes), dim=dim)


def fused_apply_rotary_pos_emb(t: torch.Tensor, freqs: torch.Tensor, transpose_output_memory: bool = False,
                               interleaved: bool = False) -> torch.Tensor:
    """Rotary embedding of ``t`` [s, b, h, d] with angles ``freqs`` [s, 1, 1, d_rot] through the native kernel
    (reference: transformer_engine.py:1602)."""
    from ..ops import core as ops
    ang = freqs.reshape(freqs.shape[0], -1).float()
    # the reference's table repeats every angle (two halves, or neighbouring pairs when interleaved); the kernel
    # takes each angle once
    ang = ang[:, 0::2] if interleaved else ang[:, : ang.shape[1] // 2]
    return ops.apply_rope(t, torch.cos(ang).contiguous(), torch.sin(ang).contiguous(), interleaved)


def te_general_gemm(A: torch.Tensor, B: torch.Tensor, out_dtype=None, layout: str = "TN", out=None, bias=None,
                    grad: bool = False):
    """The library's general GEMM entry in its column-major convention: ``layout="TN"`` computes ``B @ A^T`` for
    row-major ``A`` [n, k], ``B`` [m, k] (reference: transformer_engine.py:1697).  Runs the native tcgen05 GEMM on a
    GPU.  Returns a list whose first entry is the product, like the library."""
    from ..ops.gemm import gemm
    if layout == "TN":
        x, w, kw = B, A, {}
    elif layout == "NN":
        x, w, kw = B, A, {"b_mn": True}
    elif layout == "NT":
        x, w, kw = B, A, {"a_mn": True, "b_mn": True}
    else:
        raise ValueError(f"layout {layout!r}")
    if x.is_cuda:
        y = gemm(x, w, bias=bias, out=out, out_dtype=out_dtype, **kw) if out_dtype is not None or out is not None \
            else gemm(x, w, bias=bias, **kw)
    else:
        xa = x.t() if kw.get("a_mn") else x
        wa = w if kw.get("b_mn") else w.t()
        y = xa.float() @ wa.float()
        if bias is not None:
            y = y + bias.float()
        y = y.to(out_dtype or x.dtype)
        if out is not None:
            out.copy_(y)
            y = out
    return [y, None, None, None]
