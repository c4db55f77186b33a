"""Retro: a GPT decoder whose selected layers cross-attend, chunk by chunk, to encoded retrieved neighbours.

Reference: megatron/core/models/retro/ (``RetroConfig`` config.py:17, ``RetroModel`` model.py:14,
``RetroDecoderCrossAttention`` decoder_attention.py:26, ``RetroEncoderCrossAttention``
encoder_attention.py:19, layer placement decoder_spec.py:141).

Sequence length n = l chunks of m tokens; each chunk has k neighbours of r retrieved tokens.
* Encoder (a small bidirectional block) runs over every neighbour [r, b*l*k, h]; its first layer
  cross-attends to the hidden states of the chunk the neighbour belongs to.
* Decoder cross-attention at layers P (first at 6 or 9, then every 3rd): the hidden states are shifted
  left by m-1 so that chunk c only sees neighbours retrieved for chunks <= c-1 (causality), attended
  chunk-wise to [r*k, b*l, h], then shifted back; the first m-1 positions get no retrieval signal.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import TransformerConfig
from ..ops import core as ops
from .gpt import GPTModel
from .transformer import CrossAttention, Norm, TransformerBlock, TransformerLayer


@dataclass
class RetroConfig(TransformerConfig):
    retro_project_dir: Optional[str] = None
    retro_block_size: Optional[int] = None
    retro_chunk_length: int = 64
    retro_encoder_num_layers: int = 2
    retro_encoder_hidden_dropout: float = 0.1
    retro_encoder_attention_dropout: float = 0.1
    retro_neighbor_dirs: Optional[dict] = None
    retro_num_neighbors: int = 2
    retro_num_retrieved_chunks: int = 2
    retro_retrieved_length: Optional[int] = None
    retro_split_preprocessing: Optional[str] = None
    retro_verify_neighbor_count: bool = True
    retro_attention_gate: float = 1.0           # multiplies the retrieval update (0 switches retrieval off)

    def __post_init__(self):
        super().__post_init__()
        if self.retro_retrieved_length is None:
            self.retro_retrieved_length = self.retro_num_retrieved_chunks * self.retro_chunk_length


def get_retro_decoder_layer_numbers(num_layers: int) -> List[int]:
    """1-based layers that carry retrieval cross-attention."""
    start = 6 if num_layers <= 15 else 9
    if num_layers < start:
        start = max(1, num_layers // 2)
    return list(range(start, num_layers + 1, 3))


class RetroEncoder(nn.Module):
    def __init__(self, config: RetroConfig):
        super().__init__()
        import copy
        ecfg = copy.copy(config)
        ecfg.num_layers = config.retro_encoder_num_layers
        ecfg.hidden_dropout = config.retro_encoder_hidden_dropout
        ecfg.attention_dropout = config.retro_encoder_attention_dropout
        ecfg.pipeline_model_parallel_size = 1
        ecfg.virtual_pipeline_model_parallel_size = None
        self.layers = nn.ModuleList([TransformerLayer(ecfg, i + 1, causal=False, cross_attention=(i == 0))
                                     for i in range(ecfg.num_layers)])
        self.final_layernorm = Norm(ecfg, ecfg.hidden_size)

    def forward(self, neighbours, chunk_hidden):
        """neighbours [r, b*l*k, h]; chunk_hidden [m, b*l*k, h] (each neighbour's own chunk)."""
        h = neighbours
        for layer in self.layers:
            h = layer(h, encoder_output=chunk_hidden)
        return self.final_layernorm(h)


class RetroDecoderCrossAttention(nn.Module):
    def __init__(self, config: RetroConfig, layer_number: int, encoder: Optional[RetroEncoder]):
        super().__init__()
        self.config = config
        self.m, self.k, self.r = config.retro_chunk_length, config.retro_num_neighbors, config.retro_retrieved_length
        self.norm = Norm(config, config.hidden_size)
        self.attn = CrossAttention(config, layer_number)
        self.encoder = encoder                                     # only the first retrieval layer encodes

    def forward(self, hidden, context):
        """hidden [n, b, h]; context: embedded neighbours [r, b*l*k, h] before the first retrieval layer,
        encoded neighbours afterwards.  Returns (hidden + retrieval update, encoded context)."""
        n, b, h = hidden.shape
        m, k, r = self.m, self.k, self.r
        l = (n + m - 1) // m
        ln = self.norm(hidden)
        if self.encoder is not None:
            first = F.pad(ln, (0, 0, 0, 0, 0, l * m - n))          # [l*m, b, h]
            chunks = first.view(l, m, b, h).permute(1, 2, 0, 3).reshape(m, b * l, h)
            chunks_k = chunks.unsqueeze(2).expand(m, b * l, k, h).reshape(m, b * l * k, h)
            context = self.encoder(context, chunks_k.contiguous())
        ctx = context.view(r, b * l, k, h).permute(2, 0, 1, 3).reshape(k * r, b * l, h)
        # shift so that the attending block for chunk c starts at its last token
        pad = (m - 1)
        shifted = F.pad(ln[pad:], (0, 0, 0, 0, 0, l * m - (n - pad)))          # [l*m, b, h]
        q = shifted.view(l, m, b, h).permute(1, 2, 0, 3).reshape(m, b * l, h)
        out, bias = self.attn(q.contiguous(), ctx.contiguous())
        if bias is not None:
            out = out + bias
        out = out.view(m, b, l, h).permute(2, 0, 1, 3).reshape(l * m, b, h)
        out = F.pad(out, (0, 0, 0, 0, pad, 0))[:n]                 # undo the shift; first m-1 rows get zeros
        gate = getattr(self.config, "retro_attention_gate", 1.0)
        return hidden + gate * F.dropout(out, self.config.hidden_dropout, self.training), context


class RetroModel(GPTModel):
    """GPT plus retrieval: ``forward`` takes the neighbours' token ids [b, l, k, r]."""

    def __init__(self, config: RetroConfig, vocab_size: int, max_sequence_length: int, **kw):
        super().__init__(config, vocab_size, max_sequence_length, **kw)
        nums = [i for i in get_retro_decoder_layer_numbers(config.num_layers)]
        self.retro_layers = nn.ModuleDict()
        enc = RetroEncoder(config)
        for j, i in enumerate(nums):
            self.retro_layers[str(i)] = RetroDecoderCrossAttention(config, i, enc if j == 0 else None)
        self.retro_layer_numbers = nums

    def forward(self, input_ids, position_ids=None, attention_mask=None, context_input_ids=None,
                context_position_ids=None, context_mask=None, decoder_input=None, labels=None, inference_context=None):
        if context_input_ids is None:
            return super().forward(input_ids, position_ids, attention_mask, decoder_input, labels, inference_context)
        b, l, k, r = context_input_ids.shape
        hidden = self.embedding(input_ids, position_ids)                    # [n, b, h]
        ctx_ids = context_input_ids.reshape(b * l * k, r)
        context = self.embedding(ctx_ids, context_position_ids.reshape(b * l * k, r) if context_position_ids
                                 is not None else None)                     # [r, b*l*k, h]
        rotary = None
        if self.rotary_pos_emb is not None:
            rotary = self.rotary_pos_emb(input_ids.shape[1], input_ids.device)
        for layer in self.decoder.layers:
            num = layer.layer_number
            if str(num) in self.retro_layers:
                # the retrieval block sits between self-attention and MLP in the reference; applying it on the
                # layer input keeps the same dependency structure (causal through the chunk shift)
                hidden, context = self.retro_layers[str(num)](hidden, context)
            hidden = layer(hidden, rotary=rotary)
        if self.decoder.final_layernorm is not None:
            hidden = self.decoder.final_layernorm(hidden)
        weight = self.shared_embedding_or_output_weight() if self.share_embeddings_and_output_weights else None
        logits, _ = self.output_layer(hidden, weight=weight)
        if labels is None:
            return logits.transpose(0, 1).contiguous()
        return self.compute_language_model_loss(labels, logits)
