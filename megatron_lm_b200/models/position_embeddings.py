"""Further position encodings: T5-style relative position bias and multimodal (sectioned) rotary embedding.

Reference: megatron/core/models/common/embeddings/relative_pos_embedding.py (``RelativePositionEmbedding`` :21,
bucket rule :78) and rotary_pos_embedding.py (``MultimodalRotaryEmbedding`` :233: temporal / height / width
position ids each drive a section of the rotary channels).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn


class RelativePositionEmbedding(nn.Module):
    """Learned bias per (relative-position bucket, head), added to attention scores: [1, heads, q, k]."""

    def __init__(self, bidirectional: bool, num_attention_heads: int, relative_attention_num_buckets: int = 32,
                 relative_attention_max_distance: int = 128, init_std: float = 0.02):
        super().__init__()
        self.bidirectional = bidirectional
        self.num_buckets, self.max_distance = relative_attention_num_buckets, relative_attention_max_distance
        self.relative_attention_bias = nn.Embedding(self.num_buckets, num_attention_heads)
        nn.init.normal_(self.relative_attention_bias.weight, std=init_std)

    def _bucket(self, rel: torch.Tensor) -> torch.Tensor:
        nb = self.num_buckets
        out = torch.zeros_like(rel)
        if self.bidirectional:
            nb //= 2
            out = out + (rel > 0).long() * nb
            rel = rel.abs()
        else:
            rel = -torch.min(rel, torch.zeros_like(rel))
        exact = nb // 2
        small = rel < exact
        large = exact + (torch.log(rel.float().clamp(min=1) / exact) / math.log(self.max_distance / exact)
                         * (nb - exact)).long()
        large = torch.min(large, torch.full_like(large, nb - 1))
        return out + torch.where(small, rel, large)

    def forward(self, query_seq_length: int, key_seq_length: int) -> torch.Tensor:
        dev = self.relative_attention_bias.weight.device
        q = torch.arange(query_seq_length, device=dev)[:, None]
        k = torch.arange(key_seq_length, device=dev)[None, :]
        bias = self.relative_attention_bias(self._bucket(k - q))                 # [q, k, heads]
        return bias.permute(2, 0, 1).unsqueeze(0)


class MultimodalRotaryEmbedding(nn.Module):
    """cos/sin from three position-id streams (temporal, height, width); ``mrope_section`` gives how many of the
    rot/2 frequency channels follow each stream.  position_ids [3, b, s] -> cos, sin [s, b, rot/2]."""

    def __init__(self, kv_channels: int, rotary_percent: float = 1.0, rotary_base: float = 10000.0,
                 seq_len_interpolation_factor: Optional[float] = None):
        super().__init__()
        self.dim = int(kv_channels * rotary_percent)
        self.base, self.interp = rotary_base, seq_len_interpolation_factor

    def forward(self, position_ids: torch.Tensor, mrope_section: List[int]):
        if sum(mrope_section) != self.dim // 2:
            raise ValueError("mrope_section must sum to half the rotary dimension")
        dev = position_ids.device
        inv = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, dtype=torch.float32, device=dev) / self.dim))
        pos = position_ids.float()
        if self.interp:
            pos = pos / self.interp
        ang = pos.unsqueeze(-1) * inv                                            # [3, b, s, rot/2]
        pieces, o = [], 0
        for i, n in enumerate(mrope_section):
            pieces.append(ang[i % 3, :, :, o:o + n])
            o += n
        a = torch.cat(pieces, dim=-1).transpose(0, 1)                            # [s, b, rot/2]
        return a.cos().contiguous(), a.sin().contiguous()


def get_pos_emb_on_this_cp_rank(pos_emb: torch.Tensor, seq_dim: int, cp_size: int = None, cp_rank: int = None):
    """The rows of a full-sequence position table that this context-parallel rank holds: the sequence is cut into
    2 x cp chunks and rank r keeps chunks r and 2 cp - 1 - r, which balances causal attention work
    (reference: megatron/core/models/common/embeddings/rope_utils.py:48)."""
    from ..parallel import state
    from ..parallel.context_parallel import zigzag_indices
    if cp_size is None:
        cp_size = state.get_context_parallel_world_size() if state.model_parallel_is_initialized() else 1
    if cp_size == 1:
        return pos_emb
    if cp_rank is None:
        cp_rank = state.get_context_parallel_rank()
    idx = zigzag_indices(pos_emb.shape[seq_dim], cp_size, cp_rank, pos_emb.device)
    return pos_emb.index_select(seq_dim, idx)
