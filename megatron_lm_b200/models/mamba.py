"""Mamba-2 / hybrid state-space language model.

Reference: megatron/core/ssm/mamba_mixer.py (``MambaMixer`` :93, forward :381, ``step`` :549),
mamba_layer.py:50, mamba_block.py:91 (``MambaStack``), mamba_hybrid_layer_allocation.py:84 and
models/mamba/mamba_model.py:21.  Layer pattern symbols: ``M`` state-space mixer, ``*`` attention,
``-`` MLP.  Heads (and B/C groups) are split over tensor-parallel ranks: in_proj is column-parallel
over [z | x | B | C | dt], out_proj row-parallel.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import TransformerConfig
from ..ops import core as ops
from ..ops.mamba import causal_conv1d, causal_conv1d_update, gated_rmsnorm, ssd_scan
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, _device
from .gpt import LanguageModelEmbedding, RotaryEmbedding
from .transformer import MLP, Norm, SelfAttention


class Symbols:
    MAMBA, ATTENTION, MLP = "M", "*", "-"
    VALID = {"M", "*", "-"}


def allocate_layers(total: int, attention_ratio: float = 0.0, mlp_ratio: float = 0.0,
                    override_pattern: Optional[str] = None) -> List[str]:
    """Spread attention and MLP layers evenly among mixer layers; an explicit pattern wins."""
    if override_pattern:
        layers = list(override_pattern)
        if len(layers) != total or any(c not in Symbols.VALID for c in layers):
            raise ValueError("hybrid override pattern must have one of 'M', '*', '-' per layer")
        return layers
    n_attn = round(total * attention_ratio)
    n_mlp = round(total * mlp_ratio)
    layers = [Symbols.MAMBA] * total
    if n_attn:
        step = total / n_attn
        for i in range(n_attn):
            layers[min(int(step * i + step / 2), total - 1)] = Symbols.ATTENTION
    if n_mlp:
        free = [i for i, c in enumerate(layers) if c == Symbols.MAMBA]
        step = len(free) / n_mlp
        for i in range(n_mlp):
            layers[free[min(int(step * i + step / 2), len(free) - 1)]] = Symbols.MLP
    return layers


class MambaMixer(nn.Module):
    def __init__(self, config: TransformerConfig, layer_number: int, d_state: int = 128, d_conv: int = 4,
                 expand: int = 2, headdim: int = 64, ngroups: int = 8, dt_min=0.001, dt_max=0.1, dt_init_floor=1e-4,
                 chunk_size: int = 64):
        super().__init__()
        self.config, self.layer_number = config, layer_number
        tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.tp = tp
        d_model = config.hidden_size
        self.d_inner = expand * d_model
        self.headdim, self.d_state, self.d_conv, self.chunk = headdim, d_state, d_conv, chunk_size
        self.nheads = self.d_inner // headdim
        self.ngroups = ngroups
        if self.nheads % tp or ngroups % tp or self.nheads % ngroups:
            raise ValueError("heads and groups must divide by the tensor-parallel size, and heads by groups")
        self.h_loc, self.g_loc, self.di_loc = self.nheads // tp, ngroups // tp, self.d_inner // tp
        # in_proj rows are laid out per rank as [z | x | B | C | dt]
        in_out = 2 * self.d_inner + 2 * ngroups * d_state + self.nheads
        self.in_proj = ColumnParallelLinear(d_model, in_out, config=config, init_method=config.init_method, bias=False)
        conv_dim = self.di_loc + 2 * self.g_loc * d_state
        dev, dt_ = _device(config), config.params_dtype
        self.conv_weight = nn.Parameter(torch.empty(conv_dim, d_conv, device=dev, dtype=dt_))
        self.conv_bias = nn.Parameter(torch.zeros(conv_dim, device=dev, dtype=dt_))
        nn.init.uniform_(self.conv_weight, -1 / math.sqrt(d_conv), 1 / math.sqrt(d_conv))
        dt0 = torch.exp(torch.rand(self.h_loc, device=dev) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        dt0 = dt0.clamp(min=dt_init_floor)
        self.dt_bias = nn.Parameter((dt0 + torch.log(-torch.expm1(-dt0))).float())           # inverse softplus
        self.A_log = nn.Parameter(torch.log(torch.empty(self.h_loc, device=dev).uniform_(1, 16)).float())
        self.D = nn.Parameter(torch.ones(self.h_loc, device=dev, dtype=torch.float32))
        self.norm_weight = nn.Parameter(torch.ones(self.di_loc, device=dev, dtype=dt_))
        for p in (self.conv_weight, self.conv_bias, self.dt_bias, self.A_log, self.D, self.norm_weight):
            p.tensor_model_parallel = True
            p.partition_dim = 0
        self.dt_bias._no_weight_decay = self.A_log._no_weight_decay = self.D._no_weight_decay = True
        # a sharded checkpoint stores every segment as a tensor of its own, so the tensor-parallel size can change
        seg = [self.di_loc, self.di_loc, self.g_loc * d_state, self.g_loc * d_state, self.h_loc]
        self.in_proj.weight.partition_sizes, self.in_proj.weight.partition_names = seg, ["z", "x", "B", "C", "dt"]
        for p in (self.conv_weight, self.conv_bias):
            p.partition_sizes, p.partition_names = seg[1:4], ["x", "B", "C"]
        self.out_proj = RowParallelLinear(self.d_inner, d_model, config=config,
                                          init_method=config.output_layer_init_method, bias=False, skip_bias_add=True)
        self.eps = config.layernorm_epsilon
        # context parallelism: the convolution and the scan need the whole sequence, so the mixer trades its
        # sequence shard for a head shard (all-to-all over the context-parallel group), runs on all positions of
        # 1 / cp of its heads and groups, and trades back (reference: megatron/core/ssm/mamba_context_parallel.py:17)
        self.cp = state.get_context_parallel_world_size() if state.model_parallel_is_initialized() else 1
        if self.cp > 1 and (self.h_loc % self.cp or self.g_loc % self.cp):
            raise ValueError("Mamba heads and groups per tensor-parallel rank must divide by the context-parallel size")

    # -- context parallel <-> head parallel -------------------------------------------------------------------------
    def _cp_parts(self, xBC, dt):
        """Channel pieces that go to each context-parallel rank: its heads of x and dt, its groups of B and C."""
        cp, di, gn = self.cp, self.di_loc, self.g_loc * self.d_state
        x, Bm, Cm = torch.split(xBC, [di, gn, gn], dim=-1)
        return [torch.cat((xx, bb, cc, dd), dim=-1)
                for xx, bb, cc, dd in zip(x.chunk(cp, -1), Bm.chunk(cp, -1), Cm.chunk(cp, -1), dt.chunk(cp, -1))]

    def _cp_to_heads(self, xBC, dt):
        """[b, s/cp, channels] on every rank -> [b, s, channels/cp] in natural token order."""
        from ..parallel.context_parallel import natural_order_permutation
        from ..parallel.mappings import all_to_all
        cp, group = self.cp, state.get_context_parallel_group()
        b, sl, _ = xBC.shape
        send = torch.stack(self._cp_parts(xBC, dt), dim=0)                      # [cp (destination), b, s/cp, c]
        c = send.shape[-1]
        recv = all_to_all(group, send.reshape(cp * b * sl, c)).view(cp, b, sl, c)  # [cp (source), ...]
        seq = recv.permute(1, 0, 2, 3).reshape(b, cp * sl, c)                    # rank-concatenated zig-zag order
        seq = seq.index_select(1, natural_order_permutation(cp * sl, cp, seq.device))
        di, gn, h = self.di_loc // cp, self.g_loc * self.d_state // cp, self.h_loc // cp
        x, Bm, Cm, dtp = torch.split(seq, [di, gn, gn, h], dim=-1)
        return torch.cat((x, Bm, Cm), dim=-1), dtp

    def _heads_to_cp(self, y):
        """[b, s, channels/cp] in natural order -> this rank's [b, s/cp, channels]."""
        from ..parallel.context_parallel import zigzag_indices
        from ..parallel.mappings import all_to_all
        cp, group = self.cp, state.get_context_parallel_group()
        b, S, c = y.shape
        order = torch.cat([zigzag_indices(S, cp, r, y.device) for r in range(cp)])
        send = y.index_select(1, order).view(b, cp, S // cp, c).permute(1, 0, 2, 3).contiguous()
        recv = all_to_all(group, send.reshape(cp * b * (S // cp), c)).view(cp, b, S // cp, c)   # [cp (head part), ...]
        return recv.permute(1, 2, 0, 3).reshape(b, S // cp, cp * c)

    def _cp_params(self):
        """This context-parallel rank's rows of the convolution and its heads' scan parameters."""
        cp, r = self.cp, state.get_context_parallel_rank()
        di, gn = self.di_loc, self.g_loc * self.d_state

        def conv_rows(p):
            x, Bm, Cm = torch.split(p, [di, gn, gn], dim=0)
            return torch.cat((x.chunk(cp, 0)[r], Bm.chunk(cp, 0)[r], Cm.chunk(cp, 0)[r]), dim=0)
        return (conv_rows(self.conv_weight), conv_rows(self.conv_bias), self.dt_bias.chunk(cp)[r],
                self.A_log.chunk(cp)[r], self.D.chunk(cp)[r])

    def _split(self, zxbcdt):
        di, gn = self.di_loc, self.g_loc * self.d_state
        return torch.split(zxbcdt, [di, di + 2 * gn, self.h_loc], dim=-1)

    def _gated_norm(self, y, z):
        """RMSNorm(y * silu(z)) per tensor-parallel group of channels (reference: ssm/mamba_mixer.py:52)."""
        return gated_rmsnorm(y, z, self.norm_weight, self.g_loc, self.eps)

    def forward(self, hidden_states, inference_context=None):
        """hidden_states [s, b, h] -> ([s, b, h], None)."""
        zxbcdt, _ = self.in_proj(hidden_states)                       # [s, b, local]
        zxbcdt = zxbcdt.transpose(0, 1)                                # [b, s, local]
        z, xBC, dt = self._split(zxbcdt)
        cache = None if inference_context is None else inference_context.ssm_cache(self.layer_number, self, zxbcdt)
        if self.cp > 1:
            if cache is not None:
                raise NotImplementedError("token-by-token decoding of a context-parallel Mamba model")
            return self._forward_context_parallel(z, xBC, dt)
        b, s, _ = xBC.shape
        if cache is not None and s == 1 and cache["filled"]:
            xBC = causal_conv1d_update(xBC[:, 0], cache["conv"], self.conv_weight, self.conv_bias, True).unsqueeze(1)
        else:
            if cache is not None:
                k = self.d_conv - 1
                tail = xBC[:, -k:] if s >= k else F.pad(xBC, (0, 0, k - s, 0))
                cache["conv"].copy_(tail)
            xBC = causal_conv1d(xBC.contiguous(), self.conv_weight, self.conv_bias, True)
        gn = self.g_loc * self.d_state
        x, Bm, Cm = torch.split(xBC, [self.di_loc, gn, gn], dim=-1)
        x = x.reshape(b, s, self.h_loc, self.headdim)
        Bm = Bm.reshape(b, s, self.g_loc, self.d_state)
        Cm = Cm.reshape(b, s, self.g_loc, self.d_state)
        dtv = F.softplus(dt.float() + self.dt_bias)
        A = -torch.exp(self.A_log.float())
        if cache is not None:
            y = ssd_scan(x, dtv, A, Bm, Cm, self.D, None, cache["ssm"], cache["filled"], self.chunk)
            cache["filled"] = True
        else:
            y = ssd_scan(x, dtv, A, Bm, Cm, self.D, None, None, False, self.chunk)
        y = self._gated_norm(y.reshape(b, s, self.di_loc), z)
        return self.out_proj(y.transpose(0, 1).contiguous())


def _mixer_forward_context_parallel(self, z, xBC, dt):
    cp = self.cp
    xBC, dt = self._cp_to_heads(xBC, dt)                                     # all positions, 1 / cp of the heads
    conv_w, conv_b, dt_bias, A_log, D = self._cp_params()
    b, s, _ = xBC.shape
    h, g, di = self.h_loc // cp, self.g_loc // cp, self.di_loc // cp
    xBC = causal_conv1d(xBC.contiguous(), conv_w.contiguous(), conv_b.contiguous(), True)
    gn = g * self.d_state
    x, Bm, Cm = torch.split(xBC, [di, gn, gn], dim=-1)
    dtv = F.softplus(dt.float() + dt_bias)
    A = -torch.exp(A_log.float())
    y = ssd_scan(x.reshape(b, s, h, self.headdim), dtv, A, Bm.reshape(b, s, g, self.d_state),
                 Cm.reshape(b, s, g, self.d_state), D, None, None, False, self.chunk)
    y = self._heads_to_cp(y.reshape(b, s, di))                               # this rank's positions, all local heads
    y = self._gated_norm(y, z)
    return self.out_proj(y.transpose(0, 1).contiguous())


MambaMixer._forward_context_parallel = _mixer_forward_context_parallel


class MambaLayer(nn.Module):
    """x + mixer(norm(x))."""

    def __init__(self, config, layer_number, **mixer_kw):
        super().__init__()
        self.norm = Norm(config, config.hidden_size)
        self.mixer = MambaMixer(config, layer_number, **mixer_kw)
        self.dropout = config.hidden_dropout

    def forward(self, h, inference_context=None, **_):
        out, bias = self.mixer(self.norm(h), inference_context=inference_context)
        return ops.bias_dropout_add(out, bias, h, self.dropout, self.training)


class _AttnLayer(nn.Module):
    def __init__(self, config, layer_number):
        super().__init__()
        self.input_layernorm = Norm(config, config.hidden_size)
        self.self_attention = SelfAttention(config, layer_number)
        self.dropout = config.hidden_dropout

    def forward(self, h, rotary=None, inference_context=None, **_):
        out, bias = self.self_attention(self.input_layernorm(h), rotary=rotary, inference_context=inference_context)
        return ops.bias_dropout_add(out, bias, h, self.dropout, self.training)


class _MLPLayer(nn.Module):
    def __init__(self, config, layer_number):
        super().__init__()
        self.pre_mlp_layernorm = Norm(config, config.hidden_size)
        self.mlp = MLP(config)
        self.dropout = config.hidden_dropout

    def forward(self, h, **_):
        out, bias = self.mlp(self.pre_mlp_layernorm(h))
        return ops.bias_dropout_add(out, bias, h, self.dropout, self.training)


class MambaStack(nn.Module):
    def __init__(self, config, pre_process=True, post_process=True, hybrid_attention_ratio=0.0, hybrid_mlp_ratio=0.0,
                 hybrid_override_pattern=None, post_layer_norm=True, **mixer_kw):
        super().__init__()
        self.config, self.pre_process, self.post_process = config, pre_process, post_process
        pattern = allocate_layers(config.num_layers, hybrid_attention_ratio, hybrid_mlp_ratio, hybrid_override_pattern)
        pp = state.get_pipeline_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        rank = state.get_pipeline_model_parallel_rank() if pp > 1 else 0
        per = config.num_layers // pp
        self.layer_types = pattern[rank * per:(rank + 1) * per]
        mk = {"M": lambda i: MambaLayer(config, i, **mixer_kw), "*": lambda i: _AttnLayer(config, i),
              "-": lambda i: _MLPLayer(config, i)}
        self.layers = nn.ModuleList([mk[t](rank * per + i + 1) for i, t in enumerate(self.layer_types)])
        self.final_norm = Norm(config, config.hidden_size) if (post_process and post_layer_norm) else None
        self.input_tensor = None

    def set_input_tensor(self, t):
        self.input_tensor = t

    def forward(self, h, rotary=None, inference_context=None):
        if not self.pre_process and self.input_tensor is not None:
            h = self.input_tensor
        for layer in self.layers:
            h = layer(h, rotary=rotary, inference_context=inference_context)
        return self.final_norm(h) if self.final_norm is not None else h


class MambaModel(nn.Module):
    def __init__(self, config: TransformerConfig, vocab_size: int, max_sequence_length: int, pre_process=True,
                 hybrid_attention_ratio: float = 0.0, hybrid_mlp_ratio: float = 0.0,
                 hybrid_override_pattern: Optional[str] = None, post_process=True, fp16_lm_cross_entropy=False,
                 parallel_output=True, share_embeddings_and_output_weights=False,
                 position_embedding_type: str = "none", rotary_percent=1.0, rotary_base=10000.0,
                 mamba_stack_spec=None, **mixer_kw):
        super().__init__()
        self.config, self.vocab_size = config, vocab_size
        self.pre_process, self.post_process = pre_process, post_process
        self.share_embeddings_and_output_weights = share_embeddings_and_output_weights
        self.parallel_output = parallel_output
        tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.tp_size, self.tp_rank = tp, (state.get_tensor_model_parallel_rank() if tp > 1 else 0)
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, vocab_size, max_sequence_length, position_embedding_type)
        self.rotary_pos_emb = RotaryEmbedding(config.kv_channels, rotary_percent, rotary_base) \
            if position_embedding_type == "rope" else None
        self.decoder = MambaStack(config, pre_process, post_process, hybrid_attention_ratio, hybrid_mlp_ratio,
                                  hybrid_override_pattern, **mixer_kw)
        if post_process:
            self.output_layer = ColumnParallelLinear(config.hidden_size, vocab_size, config=config,
                                                     init_method=config.init_method, bias=False,
                                                     skip_weight_param_allocation=pre_process and share_embeddings_and_output_weights)
        if share_embeddings_and_output_weights and pre_process and post_process:
            self.embedding.word_embeddings.weight.expected_grad_signals = 2

    def set_input_tensor(self, t):
        if isinstance(t, (list, tuple)):
            t = t[0]
        self.decoder.set_input_tensor(t)

    def forward(self, input_ids, position_ids=None, attention_mask=None, decoder_input=None, labels=None,
                inference_context=None):
        span = None
        if inference_context is not None and hasattr(inference_context, "rope_span"):
            # a generation step of an engine: (positions covered, first position) for attention layers of hybrids
            span = inference_context.rope_span(input_ids)
            if position_ids is None:
                position_ids = (torch.arange(input_ids.shape[1], device=input_ids.device) + span[1]).unsqueeze(0)
        if decoder_input is None and self.pre_process:
            decoder_input = self.embedding(input_ids, position_ids)
        rotary = None
        if self.rotary_pos_emb is not None:
            rotary = self.rotary_pos_emb(input_ids.shape[1], input_ids.device) if span is None else \
                self.rotary_pos_emb(span[0], input_ids.device, span[1])
            cp = state.get_context_parallel_world_size() if state.model_parallel_is_initialized() else 1
            if cp > 1 and span is None:
                # attention layers of a hybrid under context parallelism: the table is built for the whole sequence
                # and holds the rows of this rank's two chunks
                rotary = self.rotary_pos_emb(input_ids.shape[1] * cp, input_ids.device)
        h = self.decoder(decoder_input, rotary=rotary, inference_context=inference_context)
        if not self.post_process:
            return h
        w = self.embedding.word_embeddings.weight if (self.share_embeddings_and_output_weights and self.pre_process) else None
        logits, _ = self.output_layer(h, weight=w)
        if labels is None:
            return logits.transpose(0, 1).contiguous()
        tgt = labels.transpose(0, 1).contiguous()
        group = state.get_tensor_model_parallel_group() if self.tp_size > 1 else None
        if not logits.is_cuda:
            logits = logits.float()
        loss = ops.cross_entropy(logits, tgt, vocab_start=self.tp_rank * logits.shape[-1], vocab_total=self.vocab_size,
                                 group=group)
        return loss.transpose(0, 1).contiguous()


class MambaInferenceCache:
    """Per-layer convolution window and state-space state for token-by-token decoding."""

    def __init__(self):
        self.layers = {}

    def ssm_cache(self, layer_number, mixer: MambaMixer, like):
        if layer_number not in self.layers:
            b = like.shape[0]
            conv_dim = mixer.di_loc + 2 * mixer.g_loc * mixer.d_state
            self.layers[layer_number] = {
                "conv": torch.zeros(b, mixer.d_conv - 1, conv_dim, dtype=like.dtype, device=like.device),
                "ssm": torch.zeros(b, mixer.h_loc, mixer.headdim, mixer.d_state, dtype=torch.float32, device=like.device),
                "filled": False}
        return self.layers[layer_number]
