"""T5 encoder-decoder language model.

Reference: megatron/core/models/T5/t5_model.py (``T5LMHead`` :27, ``T5Model`` :82, forward :268,
mask helpers :430-520).  Encoder layers are bidirectional; decoder layers have causal self-attention
and cross-attention over the encoder output; embeddings are shared between encoder, decoder and head.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..config import TransformerConfig
from ..ops import core as ops
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear
from .gpt import LanguageModelEmbedding, RotaryEmbedding
from .transformer import TransformerBlock


def t5_extended_attention_mask(masks):
    """Each [b, sq, sk] 1 = attend -> [b, 1, sq, sk] bool True = masked."""
    return [None if m is None else (m.unsqueeze(1) < 0.5) for m in masks]


def t5_position_ids(token_ids):
    return torch.arange(token_ids.shape[1], device=token_ids.device).unsqueeze(0).expand_as(token_ids)


class T5LMHead(nn.Module):
    def __init__(self, config, parallel_output, vocab_size, pre_process, share):
        super().__init__()
        self.parallel_output = parallel_output
        self.output_layer = ColumnParallelLinear(config.hidden_size, vocab_size, config=config,
                                                 init_method=config.init_method, bias=share,
                                                 skip_weight_param_allocation=pre_process and share)

    def forward(self, h, word_embeddings_weight):
        logits, _ = self.output_layer(h, weight=word_embeddings_weight)
        return logits


class T5Model(nn.Module):
    def __init__(self, config: TransformerConfig, encoder_config: Optional[TransformerConfig] = None,
                 vocab_size: int = 0, max_sequence_length: int = 512, pre_process: bool = True,
                 post_process: bool = True, fp16_lm_cross_entropy: bool = False, parallel_output: bool = True,
                 share_embeddings_and_output_weights: bool = True, position_embedding_type: str = "learned_absolute",
                 rotary_percent: float = 1.0, add_encoder: bool = True, add_decoder: bool = True,
                 transformer_encoder_layer_spec=None, transformer_decoder_layer_spec=None,
                 seq_len_interpolation_factor=None, vp_stage=None):
        super().__init__()
        self.config = config
        self.encoder_config = encoder_config or config
        self.vocab_size = vocab_size
        self.pre_process, self.post_process = pre_process, post_process
        self.add_encoder, self.add_decoder = add_encoder, add_decoder
        self.share_embeddings_and_output_weights = share_embeddings_and_output_weights
        tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.tp_size, self.tp_rank = tp, (state.get_tensor_model_parallel_rank() if tp > 1 else 0)
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, vocab_size, max_sequence_length, position_embedding_type)
        self.rotary_pos_emb = RotaryEmbedding(config.kv_channels, rotary_percent, 10000.0,
                                              seq_len_interpolation_factor) if position_embedding_type == "rope" else None
        if add_encoder:
            self.encoder = TransformerBlock(self.encoder_config, pre_process, True, vp_stage, causal=False)
        if add_decoder:
            self.decoder = TransformerBlock(config, pre_process, post_process, vp_stage, causal=True,
                                            cross_attention=True)
        if post_process:
            self.lm_head = T5LMHead(config, parallel_output, vocab_size, pre_process,
                                    share_embeddings_and_output_weights)
        if share_embeddings_and_output_weights and pre_process and post_process:
            self.embedding.word_embeddings.weight.expected_grad_signals = 2
        self.encoder_hidden_state = None

    def set_input_tensor(self, t):
        if isinstance(t, (list, tuple)):
            t = t[0]
        (self.encoder if self.add_encoder and not self.add_decoder else self.decoder).set_input_tensor(t)

    def forward(self, encoder_input_ids, decoder_input_ids, encoder_attn_mask=None, decoder_attn_mask=None,
                encoder_decoder_attn_mask=None, lm_labels=None, encoder_hidden_states=None, output_encoder_hidden_only=False):
        enc_mask, dec_mask, x_mask = t5_extended_attention_mask([encoder_attn_mask, decoder_attn_mask,
                                                                 encoder_decoder_attn_mask])
        rot_e = rot_d = None
        if self.rotary_pos_emb is not None:
            rot_e = self.rotary_pos_emb(encoder_input_ids.shape[1], encoder_input_ids.device)
            rot_d = self.rotary_pos_emb(decoder_input_ids.shape[1], decoder_input_ids.device)
        if encoder_hidden_states is None and self.add_encoder:
            x = self.embedding(encoder_input_ids, t5_position_ids(encoder_input_ids)) if self.pre_process else None
            encoder_hidden_states = self.encoder(x, rotary=rot_e, attention_mask=enc_mask)
        if not self.add_decoder or output_encoder_hidden_only:
            return encoder_hidden_states
        y = self.embedding(decoder_input_ids, t5_position_ids(decoder_input_ids)) if self.pre_process else None
        # the decoder's self-attention is causal by construction; its padding mask (if any) is combined with it
        h = self.decoder(y, rotary=rot_d, encoder_output=encoder_hidden_states, attention_mask=dec_mask,
                         enc_dec_attn_mask=x_mask)
        if not self.post_process:
            return h
        w = self.embedding.word_embeddings.weight if (self.share_embeddings_and_output_weights and self.pre_process) else None
        logits = self.lm_head(h, w)                                          # [s, b, v/tp]
        if lm_labels is None:
            return logits.transpose(0, 1).contiguous()
        tgt = lm_labels.transpose(0, 1).contiguous()
        group = state.get_tensor_model_parallel_group() if self.tp_size > 1 else None
        if not logits.is_cuda:
            logits = logits.float()
        loss = ops.cross_entropy(logits, tgt, vocab_start=self.tp_rank * logits.shape[-1], vocab_total=self.vocab_size,
                                 group=group)
        return loss.transpose(0, 1).contiguous()
