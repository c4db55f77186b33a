"""Classification fine-tuning loop pieces (reference: tasks/finetune_utils.py: ``process_batch`` :37,
``cross_entropy_loss_func`` :49, ``accuracy_func_provider`` eval_utils.py:18)."""
from __future__ import annotations

from typing import Callable, Dict, Iterable

import torch
import torch.nn.functional as F


def process_batch(batch: Dict[str, torch.Tensor], device, fp16: bool = False):
    tokens = batch["text"].long().to(device).contiguous()
    types = batch["types"].long().to(device).contiguous()
    labels = batch["label"].long().to(device).contiguous()
    mask = batch["padding_mask"].float().to(device).contiguous()
    if fp16:
        mask = mask.half()
    return tokens, types, labels, mask


def cross_entropy_loss_func(labels, output_tensor):
    logits = output_tensor.contiguous().float()
    loss = F.cross_entropy(logits, labels)
    return loss, {"lm loss": loss.detach()}


@torch.no_grad()
def calculate_correct_answers(model: Callable, loader: Iterable, device) -> Dict[str, float]:
    correct = total = 0
    for batch in loader:
        tokens, types, labels, mask = process_batch(batch, device)
        logits = model(tokens, mask, types)
        correct += int((logits.argmax(-1) == labels).sum())
        total += labels.numel()
    return {"correct": correct, "total": total, "accuracy": correct / max(total, 1)}
