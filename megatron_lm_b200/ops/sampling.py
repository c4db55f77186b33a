"""Token sampling (temperature / top-k / top-p / multinomial) as one CUDA kernel per batch of rows
(``csrc/sampling.cu``).  ``sample(logits, uniform, ...)`` draws by inverse CDF in vocabulary order from the filtered
distribution, so a given ``uniform`` vector makes the draw reproducible; CPU tensors use the PyTorch body below,
which states the same rule and is the numerical reference of the kernel.
Reference: megatron/core/inference/text_generation_controllers/text_generation_controller.py:164.
"""
from __future__ import annotations

import torch

from . import _lib

_lib.register_signatures({"mlb_sample": "ipppii" "l" "fif" "p"})


def _kept_probs(logits, temperature, top_k, top_p):
    x = logits.float() / temperature
    if top_k > 1 and top_k < x.size(-1):
        kth = torch.topk(x, top_k, dim=-1)[0][..., -1, None]
        x = x.masked_fill(x < kth, float("-inf"))
    elif top_k <= 1 and 0.0 < top_p < 1.0:
        srt, _ = torch.sort(x, descending=True, dim=-1)
        sp = srt.softmax(dim=-1)
        before = sp.cumsum(dim=-1) - sp                       # mass of the strictly more likely tokens
        keep = before <= top_p
        thr = srt.masked_fill(~keep, float("inf")).min(dim=-1, keepdim=True)[0]
        x = x.masked_fill(x < thr, float("-inf"))
    return torch.exp(x - x.max(dim=-1, keepdim=True)[0])


def sample_reference(logits, uniform, temperature=1.0, top_k=0, top_p=0.0):
    if top_k == 1:
        return torch.argmax(logits, dim=-1)
    p = _kept_probs(logits, temperature, top_k, top_p)
    cum = p.cumsum(dim=-1)
    target = uniform.float().unsqueeze(-1) * cum[..., -1:]
    tok = (cum <= target).sum(dim=-1)
    return tok.clamp(max=logits.size(-1) - 1)


def sample(logits: torch.Tensor, uniform: torch.Tensor, temperature: float = 1.0, top_k: int = 0,
           top_p: float = 0.0) -> torch.Tensor:
    """logits [rows, V], uniform [rows] in [0, 1) -> int64 token ids [rows]."""
    if top_k > logits.size(-1):
        raise ValueError("top-k is larger than the vocabulary")
    if top_p > 1.0:
        raise ValueError("top-p must be at most 1")
    if not logits.is_cuda:
        return sample_reference(logits, uniform, temperature, top_k, top_p)
    lg = logits if logits.stride(-1) == 1 and logits.dim() == 2 else logits.reshape(-1, logits.size(-1)).contiguous()
    rows, V = lg.shape
    u = uniform.to(device=lg.device, dtype=torch.float32).contiguous()
    out = torch.empty(rows, dtype=torch.int64, device=lg.device)
    _lib.check(_lib.lib().mlb_sample(_lib.dt(lg), lg.data_ptr(), u.data_ptr(), out.data_ptr(), rows, V, lg.stride(0),
                                     float(temperature), int(top_k), float(top_p), _lib.stream()), "sample")
    return out
