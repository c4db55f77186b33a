"""GPT / Llama / Mixtral-style decoder-only language model.

Public surface mirrors ``GPTModel`` of the reference
(megatron/core/models/gpt/gpt_model.py:34; forward :340; _preprocess :252;
_postprocess :411; tied embeddings via language_module.py:147) with
``pre_process`` / ``post_process`` selecting the embedding and the output layer
for pipeline stages, and ``vp_stage`` for interleaved schedules.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..config import TransformerConfig
from ..ops import core as ops
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear, VocabParallelEmbedding, _device, tp_linear
from ..parallel.mappings import scatter_to_sequence_parallel_region
from ..parallel.random import get_cuda_rng_tracker
from .transformer import TransformerBlock


class LanguageModelEmbedding(nn.Module):
    """Token (+ learned position) embeddings, returned as [s, b, h] and scattered along the
    sequence when sequence parallelism is on (reference:
    models/common/embeddings/language_model_embedding.py)."""

    def __init__(self, config: TransformerConfig, vocab_size: int, max_sequence_length: int,
                 position_embedding_type: str = "learned_absolute", num_tokentypes: int = 0):
        super().__init__()
        self.config = config
        self.add_position_embedding = position_embedding_type == "learned_absolute"
        self.word_embeddings = VocabParallelEmbedding(vocab_size, config.hidden_size,
                                                      init_method=config.embedding_init_method, config=config)
        if self.add_position_embedding:
            self.position_embeddings = nn.Embedding(max_sequence_length, config.hidden_size, device=_device(config),
                                                    dtype=config.params_dtype)
            if config.perform_initialization:
                config.embedding_init_method(self.position_embeddings.weight)
        if num_tokentypes > 0:
            self.tokentype_embeddings = nn.Embedding(num_tokentypes, config.hidden_size, device=_device(config),
                                                     dtype=config.params_dtype)
            if config.perform_initialization:
                config.embedding_init_method(self.tokentype_embeddings.weight)
        else:
            self.tokentype_embeddings = None
        self.dropout_p = config.hidden_dropout

    def forward(self, input_ids, position_ids=None, tokentype_ids=None):
        emb = self.word_embeddings(input_ids)                       # [b, s, h]
        if self.add_position_embedding:
            if position_ids is None:
                position_ids = torch.arange(input_ids.shape[1], device=input_ids.device).unsqueeze(0)
            emb = emb + self.position_embeddings(position_ids)
        if tokentype_ids is not None and self.tokentype_embeddings is not None:
            emb = emb + self.tokentype_embeddings(tokentype_ids)
        emb = emb.transpose(0, 1).contiguous()                      # [s, b, h]
        if self.config.fp32_residual_connection:
            emb = emb.float()
        if self.config.sequence_parallel:
            emb = scatter_to_sequence_parallel_region(emb)
            if self.config.clone_scatter_output_in_embedding:
                emb = emb.clone()
            if self.dropout_p > 0 and self.training:
                with get_cuda_rng_tracker().fork():
                    emb = torch.nn.functional.dropout(emb, self.dropout_p, True)
        elif self.dropout_p > 0 and self.training:
            emb = torch.nn.functional.dropout(emb, self.dropout_p, True)
        return emb


class RotaryEmbedding(nn.Module):
    """cos/sin tables for RoPE, sliced for context parallelism like the batch
    (reference: rotary_pos_embedding.py:36, rope_utils.py:48-70)."""

    def __init__(self, kv_channels: int, rotary_percent: float = 1.0, rotary_base: float = 10000.0,
                 seq_len_interpolation_factor: Optional[float] = None, rope_scaling: bool = False,
                 rope_scaling_factor: float = 8.0):
        super().__init__()
        self.dim = int(kv_channels * rotary_percent)
        self.base = rotary_base
        self.interp = seq_len_interpolation_factor
        self.rope_scaling, self.rope_scaling_factor = rope_scaling, rope_scaling_factor
        self._cache = {}

    def _inv_freq(self, device):
        inv = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, dtype=torch.float32, device=device) / self.dim))
        if self.rope_scaling:   # llama-3.1 frequency-dependent scaling
            import math
            low, high, old = 1.0, 4.0, 8192
            wl = 2 * math.pi / inv
            smooth = ((old / wl) - low) / (high - low)
            scaled = torch.where(wl > old / low, inv / self.rope_scaling_factor,
                                 torch.where(wl < old / high, inv,
                                             (1 - smooth) * inv / self.rope_scaling_factor + smooth * inv))
            inv = scaled
        return inv

    def forward(self, seq_len: int, device, offset: int = 0):
        cp = state.get_context_parallel_world_size() if state.model_parallel_is_initialized() else 1
        cp_rank = state.get_context_parallel_rank() if cp > 1 else 0
        key = (seq_len, str(device), offset, cp, cp_rank)
        if key not in self._cache:
            pos = torch.arange(seq_len, dtype=torch.float32, device=device) + offset
            if self.interp:
                pos = pos / self.interp
            if cp > 1:
                from ..parallel.context_parallel import zigzag_indices
                pos = pos[zigzag_indices(seq_len, cp, cp_rank, device)]
            ang = torch.outer(pos, self._inv_freq(device))
            self._cache = {key: (ang.cos().contiguous(), ang.sin().contiguous())}
        return self._cache[key]


class GPTModel(nn.Module):
    def __init__(self, config: TransformerConfig, vocab_size: int, max_sequence_length: int,
                 pre_process: bool = True, post_process: bool = True, fp16_lm_cross_entropy: bool = False,
                 parallel_output: bool = True, share_embeddings_and_output_weights: bool = False,
                 position_embedding_type: str = "learned_absolute", rotary_percent: float = 1.0,
                 rotary_base: float = 10000.0, rope_scaling: bool = False, rope_scaling_factor: float = 8.0,
                 seq_len_interpolation_factor: Optional[float] = None, vp_stage: Optional[int] = None,
                 transformer_layer_spec=None, scatter_embedding_sequence_parallel: bool = True):
        super().__init__()
        if not isinstance(vocab_size, int):
            # the reference's positional order: (config, transformer_layer_spec, vocab_size, max_sequence_length)
            transformer_layer_spec, vocab_size, max_sequence_length, pre_process = \
                vocab_size, max_sequence_length, pre_process, True
        self.config = config
        self.vocab_size, self.max_sequence_length = vocab_size, max_sequence_length
        self.pre_process, self.post_process, self.vp_stage = pre_process, post_process, vp_stage
        self.fp16_lm_cross_entropy = fp16_lm_cross_entropy
        self.parallel_output = parallel_output
        self.share_embeddings_and_output_weights = share_embeddings_and_output_weights
        self.position_embedding_type = position_embedding_type
        tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.tp_size = tp
        self.tp_rank = state.get_tensor_model_parallel_rank() if state.model_parallel_is_initialized() else 0
        if vocab_size % tp:
            raise ValueError("vocab_size must be padded to a multiple of the tensor-parallel size")
        # multi-token prediction embeds shifted tokens on the last stage, so that stage holds the table too
        if pre_process or (post_process and config.mtp_num_layers):
            self.embedding = LanguageModelEmbedding(config, vocab_size, max_sequence_length, position_embedding_type)
        if position_embedding_type == "rope" and getattr(config, "multi_latent_attention", False):
            from .mla import YarnRotaryEmbedding
            if config.rope_type == "yarn":
                self.rotary_pos_emb = YarnRotaryEmbedding(
                    config.qk_pos_emb_head_dim, config.rotary_base, config.rotary_scaling_factor,
                    config.original_max_position_embeddings, config.beta_fast, config.beta_slow, config.mscale,
                    config.mscale_all_dim)
            else:
                self.rotary_pos_emb = RotaryEmbedding(config.qk_pos_emb_head_dim, rotary_percent, config.rotary_base)
        elif position_embedding_type == "rope":
            self.rotary_pos_emb = RotaryEmbedding(config.kv_channels, rotary_percent, rotary_base,
                                                  seq_len_interpolation_factor, rope_scaling, rope_scaling_factor)
        else:
            self.rotary_pos_emb = None
        self.decoder = TransformerBlock(config, pre_process, post_process, vp_stage, spec=transformer_layer_spec)
        if post_process:
            if config.mtp_num_layers:
                from .mtp import MultiTokenPredictionBlock
                self.mtp = MultiTokenPredictionBlock(config, vocab_size)
            skip = pre_process and share_embeddings_and_output_weights
            self.output_layer = ColumnParallelLinear(config.hidden_size, vocab_size, config=config,
                                                     init_method=config.init_method, bias=False,
                                                     skip_weight_param_allocation=skip)
            self.output_layer.fp8_eligible = False          # the vocabulary projection stays in 16 bits
            if config.defer_embedding_wgrad_compute and self.output_layer.weight is not None and not config.mtp_num_layers:
                # the pipelined schedule runs this layer's weight-gradient GEMM when the pipeline drains
                self.output_layer.weight.defer_wgrad = True
                # several microbatches' gradients then arrive during the last one: no early release of its bucket
                self.output_layer.weight.expected_grad_signals = 2
        self._setup_shared_embeddings()
        if post_process and config.mtp_num_layers:
            # the prediction heads reuse the embedding and the output layer: several gradients per microbatch
            shared = list(self.embedding.parameters())
            if self.output_layer.weight is not None:
                shared.append(self.output_layer.weight)
            for p in shared:
                p.expected_grad_signals = max(2, getattr(p, "expected_grad_signals", 1))

    # -- tied embeddings ---------------------------------------------------
    def _setup_shared_embeddings(self):
        """Mark the tied weight(s).  When first and last stage differ, the last stage holds a
        zero-initialised copy that is summed with the first stage's weight at start-up and whose
        gradients are all-reduced over the embedding group every step."""
        if not self.share_embeddings_and_output_weights:
            return
        if self.pre_process:
            self.embedding.word_embeddings.weight.is_embedding_or_output_parameter = True
            self.embedding.word_embeddings.weight.shared_embedding = True
        if self.post_process and not self.pre_process:
            w = self.output_layer.weight
            with torch.no_grad():
                w.zero_()
            w.shared = True
            w.shared_embedding = True
            w.is_embedding_or_output_parameter = True
        if self.post_process and self.pre_process:
            self.embedding.word_embeddings.weight.expected_grad_signals = 2
            return
        if state.model_parallel_is_initialized() and state.get_pipeline_model_parallel_world_size() > 1 \
                and state.is_rank_in_embedding_group() and torch.distributed.is_initialized():
            w = self.shared_embedding_or_output_weight()
            if w is not None:
                torch.distributed.all_reduce(w.data, group=state.get_embedding_group())

    def shared_embedding_or_output_weight(self):
        if self.pre_process:
            return self.embedding.word_embeddings.weight
        if self.post_process:
            return self.output_layer.weight
        return None

    def set_input_tensor(self, input_tensor):
        if isinstance(input_tensor, (list, tuple)):
            input_tensor = input_tensor[0]
        self.decoder.set_input_tensor(input_tensor)

    # -- forward ---------------------------------------------------------------
    def forward(self, input_ids, position_ids=None, attention_mask=None, decoder_input=None, labels=None,
                inference_context=None, loss_mask=None, runtime_gather_output: Optional[bool] = None,
                packed_seq_params=None):
        cfg = self.config
        span = None
        if packed_seq_params is not None:
            # one row of documents laid end to end: attention stays inside a document, positions restart
            if inference_context is not None:
                raise ValueError("packed sequences are a training-time layout")
            if state.model_parallel_is_initialized() and state.get_context_parallel_world_size() > 1:
                raise NotImplementedError("packed sequences with context parallelism")
            ref_ids = input_ids if input_ids is not None else position_ids
            if ref_ids is None or ref_ids.shape[0] != 1:
                raise ValueError("packed sequences come as one row of tokens, [1, total]")
            total = ref_ids.shape[1]
            if ref_ids.is_cuda and attention_mask is None:
                # GPU: per-segment causal flash attention on slices of the fused QKV activation, no dense mask
                from ..packed_seq_params import PackedSegments
                attention_mask = PackedSegments(packed_seq_params.segment_bounds(total))
            else:
                seg_mask = packed_seq_params.block_mask(total, ref_ids.device)
                attention_mask = seg_mask if attention_mask is None else (attention_mask.bool() | seg_mask)
            if position_ids is None:
                position_ids = packed_seq_params.positions(total, ref_ids.device).unsqueeze(0)
        if inference_context is not None:
            span = inference_context.rope_span(input_ids)      # (positions covered, first position) of this step
            if position_ids is None:
                position_ids = (torch.arange(input_ids.shape[1], device=input_ids.device) + span[1]).unsqueeze(0)
        if decoder_input is None and self.pre_process:
            decoder_input = self.embedding(input_ids, position_ids)
        rotary = None
        if self.rotary_pos_emb is not None:
            if span is not None:
                seq, off = span
            else:
                ref = decoder_input if decoder_input is not None else self.decoder.input_tensor
                seq = ref.shape[0]
                if cfg.sequence_parallel:
                    seq *= self.tp_size
                if state.model_parallel_is_initialized():
                    seq *= state.get_context_parallel_world_size()     # tables are built for the full sequence
                off = 0
            dev = input_ids.device if input_ids is not None else ref.device
            rotary = self.rotary_pos_emb(seq, dev, off)
            if inference_context is not None and hasattr(inference_context, "select_rope"):
                rotary = inference_context.select_rope(rotary, position_ids)    # one table row per token
            if packed_seq_params is not None:
                pos = packed_seq_params.positions(rotary[0].shape[0], rotary[0].device)
                rotary = (rotary[0][pos].contiguous(), rotary[1][pos].contiguous())
        hidden = self.decoder(decoder_input, rotary=rotary, inference_context=inference_context,
                              attention_mask=attention_mask)
        if not self.post_process:
            return hidden
        weight = None
        if self.share_embeddings_and_output_weights:
            weight = self.shared_embedding_or_output_weight()
        mtp_loss = None
        if cfg.mtp_num_layers and labels is not None and self.training:
            mtp_loss = self.mtp(hidden, input_ids, position_ids, labels, loss_mask, rotary, self.embedding,
                                self.output_layer, weight, self.compute_language_model_loss)
        logits, _ = self.output_layer(hidden, weight=weight)         # [s, b, v/tp]
        if labels is None:
            gather = self.parallel_output is False if runtime_gather_output is None else runtime_gather_output
            if gather and self.tp_size > 1:
                from ..parallel.mappings import gather_from_tensor_model_parallel_region
                logits = gather_from_tensor_model_parallel_region(logits)
            return logits.transpose(0, 1).contiguous()               # [b, s, v]
        loss = self.compute_language_model_loss(labels, logits)
        if mtp_loss is not None:
            from .mtp import MTPLossAutoScaler
            loss = MTPLossAutoScaler.apply(loss, mtp_loss)
        return loss

    def compute_language_model_loss(self, labels, logits):
        """labels [b, s] -> per-token loss [b, s] (reference: language_module.py:119)."""
        tgt = labels.transpose(0, 1).contiguous()                    # [s, b]
        v_local = logits.shape[-1]
        group = state.get_tensor_model_parallel_group() if (state.model_parallel_is_initialized()
                                                            and self.tp_size > 1) else None
        if not self.fp16_lm_cross_entropy and not logits.is_cuda:
            logits = logits.float()
        loss = ops.cross_entropy(logits, tgt, vocab_start=self.tp_rank * v_local, vocab_total=self.vocab_size,
                                 group=group)
        return loss.transpose(0, 1).contiguous()
