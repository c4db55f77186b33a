"""Packed sequences: several documents laid end to end in one row of tokens ("thd" layout), told apart by their
cumulative lengths (reference: megatron/core/packed_seq_params.py:7 PackedSeqParams, used by the attention at
extensions/transformer_engine.py:876 and by the rotary embedding at models/common/embeddings/rope_utils.py:143).

A model given ``packed_seq_params`` treats every segment as its own sequence: attention never crosses a segment
boundary and rotary positions restart at each segment.  Tokens after the last boundary (padding of the row) form a
segment of their own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class PackedSeqParams:
    qkv_format: str = "thd"
    cu_seqlens_q: Optional[torch.Tensor] = None          # [n_segments + 1] int32, starts at 0
    cu_seqlens_kv: Optional[torch.Tensor] = None
    cu_seqlens_q_padded: Optional[torch.Tensor] = None   # boundaries including per-segment padding, when it differs
    cu_seqlens_kv_padded: Optional[torch.Tensor] = None
    max_seqlen_q: Optional[int] = None
    max_seqlen_kv: Optional[int] = None
    # the same boundaries as a host list, when the caller has them: lets the attention cut the row into segments
    # without reading a device tensor back
    bounds_host: Optional[list] = None

    def _bounds(self) -> torch.Tensor:
        b = self.cu_seqlens_q_padded if self.cu_seqlens_q_padded is not None else self.cu_seqlens_q
        if b is None:
            raise ValueError("packed sequences need cu_seqlens_q")
        return b.to(torch.int64)

    def segment_ids(self, total: int, device=None) -> torch.Tensor:
        """[total] index of the segment each token belongs to."""
        b = self._bounds().to(device) if device is not None else self._bounds()
        tok = torch.arange(total, device=b.device)
        return torch.bucketize(tok, b[1:], right=True)

    def positions(self, total: int, device=None) -> torch.Tensor:
        """[total] position of each token inside its segment."""
        b = self._bounds().to(device) if device is not None else self._bounds()
        seg = self.segment_ids(total, b.device)
        starts = torch.cat((b, b.new_tensor([int(b[-1])])))[seg.clamp(max=b.numel())]
        return torch.arange(total, device=b.device) - starts

    def block_mask(self, total: int, device=None) -> torch.Tensor:
        """[1, 1, total, total] bool, True where attention is NOT allowed (different segments)."""
        seg = self.segment_ids(total, device)
        return (seg.unsqueeze(0) != seg.unsqueeze(1)).view(1, 1, total, total)

    @classmethod
    def from_lengths(cls, lengths, device=None) -> "PackedSeqParams":
        ln = torch.as_tensor(lengths, dtype=torch.int32, device=device)
        cu = torch.cat((ln.new_zeros(1), ln.cumsum(0).to(torch.int32)))
        host = [int(v) for v in (lengths.tolist() if torch.is_tensor(lengths) else lengths)]
        m = max(host) if host else 0
        bounds = [0]
        for n in host:
            bounds.append(bounds[-1] + n)
        return cls("thd", cu, cu.clone(), None, None, m, m, bounds)

    def segment_bounds(self, total: int) -> list:
        """Host list [0, ..., total] of segment boundaries (tokens after the last boundary form a segment)."""
        b = self.bounds_host if self.bounds_host is not None else [int(v) for v in self._bounds().tolist()]
        b = [v for v in b if v <= total]
        if not b or b[0] != 0:
            b = [0] + b
        if b[-1] < total:
            b.append(total)
        return b


class PackedSegments:
    """What the attention layers receive in place of a dense mask for a packed row on a GPU: the host-side
    segment boundaries.  Every segment then runs as its own causal flash-attention call on a slice of the fused
    QKV activation - no [total, total] mask is ever built."""

    def __init__(self, bounds):
        self.bounds = list(bounds)

    def __len__(self):
        return len(self.bounds) - 1
