"""BERT: bidirectional encoder with masked-LM head and optional next-sentence (binary) head.

Reference: megatron/core/models/bert/bert_model.py (``BertModel`` :36, extended mask :188, forward
:262), ``BertLMHead`` bert_lm_head.py, ``Pooler`` models/bert/pooler.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..config import TransformerConfig
from ..ops import core as ops
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear, _device
from .gpt import LanguageModelEmbedding
from .transformer import Norm, TransformerBlock


def bert_extended_attention_mask(attention_mask: torch.Tensor) -> torch.Tensor:
    """[b, s] of 1 = real token -> [b, 1, s, s] bool with True = may NOT attend."""
    m = attention_mask.unsqueeze(1) * attention_mask.unsqueeze(2)       # [b, s, s]
    return (m.unsqueeze(1) < 0.5)


class BertLMHead(nn.Module):
    def __init__(self, config: TransformerConfig):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size, device=_device(config), dtype=config.params_dtype)
        if config.perform_initialization:
            config.init_method(self.dense.weight)
            nn.init.zeros_(self.dense.bias)
        self.layer_norm = Norm(config, config.hidden_size)
        for p in self.dense.parameters():
            p.sequence_parallel = config.sequence_parallel

    def forward(self, h):
        return self.layer_norm(torch.nn.functional.gelu(self.dense(h)))


class Pooler(nn.Module):
    """tanh(W h[0]) of the first token (sequence gathered first under sequence parallelism)."""

    def __init__(self, config: TransformerConfig):
        super().__init__()
        self.config = config
        self.dense = nn.Linear(config.hidden_size, config.hidden_size, device=_device(config), dtype=config.params_dtype)
        if config.perform_initialization:
            config.init_method(self.dense.weight)
            nn.init.zeros_(self.dense.bias)

    def forward(self, h, index: int = 0):
        if self.config.sequence_parallel and state.model_parallel_is_initialized() and \
                state.get_tensor_model_parallel_world_size() > 1:
            from ..parallel.mappings import gather_from_sequence_parallel_region
            h = gather_from_sequence_parallel_region(h, tensor_parallel_output_grad=False)
        return torch.tanh(self.dense(h[index]))


class BertModel(nn.Module):
    def __init__(self, config: TransformerConfig, num_tokentypes: int, vocab_size: int, max_sequence_length: int,
                 pre_process: bool = True, post_process: bool = True, fp16_lm_cross_entropy: bool = False,
                 parallel_output: bool = True, share_embeddings_and_output_weights: bool = False,
                 position_embedding_type: str = "learned_absolute", add_binary_head: bool = True,
                 return_embeddings: bool = False, vp_stage: Optional[int] = None, transformer_layer_spec=None):
        super().__init__()
        if return_embeddings and not (post_process and add_binary_head):
            raise ValueError("return_embeddings needs the pooler of the last stage")
        self.config, self.vocab_size = config, vocab_size
        self.pre_process, self.post_process = pre_process, post_process
        self.add_binary_head, self.return_embeddings = add_binary_head, return_embeddings
        self.parallel_output = parallel_output
        self.share_embeddings_and_output_weights = share_embeddings_and_output_weights
        tp = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        self.tp_size = tp
        self.tp_rank = state.get_tensor_model_parallel_rank() if tp > 1 else 0
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, vocab_size, max_sequence_length, position_embedding_type,
                                                    num_tokentypes)
        self.encoder = TransformerBlock(config, pre_process, post_process, vp_stage, causal=False)
        if post_process:
            self.lm_head = BertLMHead(config)
            skip = pre_process and share_embeddings_and_output_weights
            self.output_layer = ColumnParallelLinear(config.hidden_size, vocab_size, config=config,
                                                     init_method=config.init_method, bias=True,
                                                     skip_weight_param_allocation=skip)
            if add_binary_head:
                self.pooler = Pooler(config)
                self.binary_head = nn.Linear(config.hidden_size, 2, device=_device(config), dtype=config.params_dtype)
                if config.perform_initialization:
                    config.init_method(self.binary_head.weight)
                    nn.init.zeros_(self.binary_head.bias)
        if share_embeddings_and_output_weights and pre_process and post_process:
            self.embedding.word_embeddings.weight.expected_grad_signals = 2

    def set_input_tensor(self, t):
        if isinstance(t, (list, tuple)):
            t = t[0]
        self.encoder.set_input_tensor(t)

    def forward(self, input_ids, attention_mask, tokentype_ids=None, lm_labels=None, inference_context=None):
        ext = bert_extended_attention_mask(attention_mask)
        x = None
        if self.pre_process:
            pos = torch.arange(input_ids.shape[1], device=input_ids.device).unsqueeze(0).expand_as(input_ids)
            x = self.embedding(input_ids, pos, tokentype_ids)
        h = self.encoder(x, attention_mask=ext)
        if not self.post_process:
            return h
        binary_logits = None
        if self.add_binary_head:
            pooled = self.pooler(h, 0)
            if self.return_embeddings:
                # mean of the real tokens between [CLS] and [SEP]
                hb = h.transpose(0, 1)
                out = torch.zeros(hb.shape[0], hb.shape[2], dtype=torch.float32, device=hb.device)
                lens = attention_mask.sum(dim=1).long()
                for i in range(hb.shape[0]):
                    out[i] = hb[i, 1:max(int(lens[i]) - 1, 2)].float().mean(dim=0)
                return out
            binary_logits = self.binary_head(pooled)
        weight = self.embedding.word_embeddings.weight if (self.share_embeddings_and_output_weights
                                                           and self.pre_process) else None
        logits, _ = self.output_layer(self.lm_head(h), weight=weight)          # [s, b, v/tp]
        if lm_labels is None:
            return logits.transpose(0, 1).contiguous(), binary_logits
        tgt = lm_labels.transpose(0, 1).contiguous()
        group = state.get_tensor_model_parallel_group() if self.tp_size > 1 else None
        if not logits.is_cuda:
            logits = logits.float()
        loss = ops.cross_entropy(logits, tgt, vocab_start=self.tp_rank * logits.shape[-1], vocab_total=self.vocab_size,
                                 group=group)
        return loss.transpose(0, 1).contiguous(), binary_logits


class Classification(nn.Module):
    """Encoder + pooler + dropout + linear head over ``num_classes`` (sentence / sentence-pair classification).
    ``MultipleChoice`` scores every choice with a one-logit head and returns [batch, choices].
    Reference: megatron/legacy/model/classification.py:19-100, multiple_choice.py:19-110."""

    def __init__(self, config: TransformerConfig, num_classes: int, vocab_size: int, max_sequence_length: int,
                 num_tokentypes: int = 2, pre_process: bool = True, post_process: bool = True):
        super().__init__()
        self.config, self.num_classes = config, num_classes
        self.pre_process, self.post_process = pre_process, post_process
        if pre_process:
            self.embedding = LanguageModelEmbedding(config, vocab_size, max_sequence_length, "learned_absolute",
                                                    num_tokentypes)
        self.encoder = TransformerBlock(config, pre_process, post_process, None, causal=False)
        if post_process:
            self.pooler = Pooler(config)
            self.classification_dropout = nn.Dropout(config.hidden_dropout)
            self.classification_head = nn.Linear(config.hidden_size, num_classes, device=_device(config),
                                                 dtype=config.params_dtype)
            if config.perform_initialization:
                config.init_method(self.classification_head.weight)
                nn.init.zeros_(self.classification_head.bias)

    def set_input_tensor(self, t):
        if isinstance(t, (list, tuple)):
            t = t[0]
        self.encoder.set_input_tensor(t)

    def _encode(self, input_ids, attention_mask, tokentype_ids):
        x = None
        if self.pre_process:
            pos = torch.arange(input_ids.shape[1], device=input_ids.device).unsqueeze(0).expand_as(input_ids)
            x = self.embedding(input_ids, pos, tokentype_ids)
        return self.encoder(x, attention_mask=bert_extended_attention_mask(attention_mask))

    def forward(self, input_ids, attention_mask, tokentype_ids=None):
        h = self._encode(input_ids, attention_mask, tokentype_ids)
        if not self.post_process:
            return h
        return self.classification_head(self.classification_dropout(self.pooler(h, 0))).view(-1, self.num_classes)

    def load_pretrained_encoder(self, bert_state_dict, strict: bool = False):
        """Take embedding, encoder and pooler from a pre-trained ``BertModel`` state dict; the head stays fresh."""
        own = self.state_dict()
        take = {k: v for k, v in bert_state_dict.items() if k in own and own[k].shape == v.shape
                and not k.startswith("classification_head")}
        return self.load_state_dict(take, strict=strict)


class MultipleChoice(Classification):
    def __init__(self, config: TransformerConfig, vocab_size: int, max_sequence_length: int, num_tokentypes: int = 2,
                 pre_process: bool = True, post_process: bool = True):
        super().__init__(config, 1, vocab_size, max_sequence_length, num_tokentypes, pre_process, post_process)

    def forward(self, input_ids, attention_mask, tokentype_ids=None):
        # [batch, choices, seq] -> every choice is a row of the encoder's batch
        b, c, s = input_ids.shape
        flat = lambda t: None if t is None else t.reshape(b * c, s)
        h = self._encode(flat(input_ids), flat(attention_mask), flat(tokentype_ids))
        if not self.post_process:
            return h
        return self.classification_head(self.classification_dropout(self.pooler(h, 0))).view(b, c)


class _BertTower(nn.Module):
    """Embedding + bidirectional encoder + pooler: what one side of the biencoder needs of a BERT model."""

    def __init__(self, config: TransformerConfig, vocab_size: int, max_sequence_length: int):
        super().__init__()
        self.embedding = LanguageModelEmbedding(config, vocab_size, max_sequence_length, "learned_absolute", 2)
        self.encoder = TransformerBlock(config, True, True, None, causal=False)
        self.pooler = Pooler(config)

    def forward(self, input_ids, attention_mask, tokentype_ids=None):
        pos = torch.arange(input_ids.shape[1], device=input_ids.device).unsqueeze(0).expand_as(input_ids)
        h = self.encoder(self.embedding(input_ids, pos, tokentype_ids),
                         attention_mask=bert_extended_attention_mask(attention_mask))
        return self.pooler(h, 0)                                                 # [b, h]


class BiEncoderModel(nn.Module):
    """Two BERT towers (query, context) whose pooled [CLS] vectors are compared by inner product - the retriever
    trained by the inverse cloze task (reference: megatron/legacy/model/biencoder_model.py:57).  With
    ``shared_query_context_model`` both sides use one tower; ``projection_dim`` > 0 adds a linear projection."""

    def __init__(self, config, vocab_size: int, max_sequence_length: int, projection_dim: int = 0,
                 shared_query_context_model: bool = False):
        super().__init__()
        self.config = config
        self.query_model = _BertTower(config, vocab_size, max_sequence_length)
        self.context_model = self.query_model if shared_query_context_model else \
            _BertTower(config, vocab_size, max_sequence_length)
        self.projection = None
        if projection_dim > 0:
            self.projection = nn.Linear(config.hidden_size, projection_dim, device=_device(config),
                                        dtype=config.params_dtype)

    def set_input_tensor(self, t):
        pass

    def init_from_bert(self, bert_state_dict) -> int:
        """Start both towers from a pre-trained ``BertModel`` (embedding, encoder, pooler; the language-model and
        binary heads are dropped).  Returns how many tensors were taken (reference: biencoder_model.py:138-190
        ``init_state_dict_from_bert``)."""
        taken = 0
        for tower in {id(self.query_model): self.query_model, id(self.context_model): self.context_model}.values():
            own = tower.state_dict()
            pick = {k: v for k, v in bert_state_dict.items() if k in own and own[k].shape == v.shape}
            tower.load_state_dict(pick, strict=False)
            taken += len(pick)
        return taken

    def _embed(self, model, tokens, pad_mask, types):
        pooled = model(tokens, pad_mask, types)
        return pooled if self.projection is None else self.projection(pooled)

    def forward(self, query_tokens, query_pad_mask, query_types, context_tokens, context_pad_mask, context_types):
        q = self._embed(self.query_model, query_tokens, query_pad_mask, query_types)
        c = self._embed(self.context_model, context_tokens, context_pad_mask, context_types)
        return q, c
