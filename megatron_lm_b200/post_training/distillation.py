"""Knowledge distillation losses and the loss balancer.

Reference: megatron/post_training/algos/distillation.py (``LogitsKLLoss`` :232 with tensor-parallel
softmax statistics, ``HiddenStateCosineLoss`` :180, ``MSELoss`` :158, ``LogitsAndIntermediatesLossBalancer``
:372, projection layer :425).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class LogitsKLLoss(nn.Module):
    """KL(teacher || student) per token over a vocabulary that may be split over a tensor-parallel group:
    the soft-max normalisers are reduced over the group, so each rank only touches its vocabulary shard."""

    def __init__(self, temperature: float = 1.0, reverse: bool = False, tp_group=None):
        super().__init__()
        self.t, self.reverse, self.group = temperature, reverse, tp_group

    def _log_softmax(self, x):
        x = x.float() / self.t
        mx = x.max(dim=-1, keepdim=True).values
        if self.group is not None and dist.get_world_size(self.group) > 1:
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)
        x = x - mx
        denom = x.exp().sum(dim=-1, keepdim=True)
        if self.group is not None and dist.get_world_size(self.group) > 1:
            denom = _AllReduceSum.apply(denom, self.group)
        return x - denom.log()

    def forward(self, student_logits, teacher_logits):
        s = self._log_softmax(student_logits)
        with torch.no_grad():
            t = self._log_softmax(teacher_logits)
        if self.reverse:
            kl = (s.exp() * (s - t)).sum(dim=-1)
        else:
            kl = (t.exp() * (t - s)).sum(dim=-1)
        if self.group is not None and dist.get_world_size(self.group) > 1:
            kl = _AllReduceSum.apply(kl, self.group)
        return kl * (self.t ** 2)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class HiddenStateCosineLoss(nn.Module):
    def __init__(self, student_hidden: int, teacher_hidden: int):
        super().__init__()
        self.proj = nn.Linear(student_hidden, teacher_hidden) if student_hidden != teacher_hidden else nn.Identity()

    def forward(self, student, teacher):
        s = self.proj(student).float()
        return 1.0 - F.cosine_similarity(s, teacher.float().detach(), dim=-1)


class MSELoss(nn.Module):
    def forward(self, student, teacher):
        return F.mse_loss(student.float(), teacher.float().detach(), reduction="none").sum(dim=-1)


class LogitsAndIntermediatesLossBalancer(nn.Module):
    """total = original + kd_scale * (logits KD + intermediates rescaled to the logits loss' magnitude);
    ``skip_original_loss`` drops the first term."""

    def __init__(self, kd_loss_scale: float = 1.0, skip_original_loss: bool = False):
        super().__init__()
        self.scale, self.skip = kd_loss_scale, skip_original_loss

    def forward(self, losses: Dict[str, torch.Tensor]) -> torch.Tensor:
        original = losses.pop("original", None)
        logits = [v for k, v in losses.items() if "logits" in k.lower()]
        inter = [v for k, v in losses.items() if "logits" not in k.lower()]
        kd = sum(logits) if logits else torch.zeros(())
        if inter:
            isum = sum(inter)
            kd = kd + isum * (kd.detach() / isum.detach().clamp(min=1e-8) if logits else 1.0)
        if original is None or self.skip:
            return kd * self.scale
        dyn = original.detach() / kd.detach().clamp(min=1e-8)
        return original + kd * dyn * self.scale
