"""Accuracy evaluation of classification-style tasks over one or more validation sets, data-parallel aware.

Reference: tasks/eval_utils.py:19-182 (``accuracy_func_provider`` builds one loader per dataset and returns a
``metrics_func(model, epoch, output_predictions)``; ``calculate_correct_answers`` runs forward-only steps and
all-reduces the correct / total counts over the data-parallel group)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..parallel import state


def _dp_group():
    if dist.is_initialized() and state.model_parallel_is_initialized() and state.get_data_parallel_world_size() > 1:
        return state.get_data_parallel_group()
    return None


@torch.no_grad()
def calculate_correct_answers(name: str, model: Callable, loader, device, output_predictions: bool = False,
                              process_batch: Optional[Callable] = None):
    """Returns (correct, total) summed over the data-parallel group; with ``output_predictions`` also
    (softmaxes, labels, ids) of this rank's samples."""
    from .finetune_utils import process_batch as default_process
    process = process_batch or default_process
    was_training = getattr(model, "training", False)
    if hasattr(model, "eval"):
        model.eval()
    correct = total = 0
    softmaxes: List = []
    labels_out: List[int] = []
    ids: List[int] = []
    for batch in loader:
        tokens, types, labels, mask = process(batch, device)
        logits = model(tokens, mask, types).float()
        pred = logits.argmax(dim=-1)
        correct += int((pred == labels).sum())
        total += labels.numel()
        if output_predictions:
            softmaxes.extend(torch.softmax(logits, dim=-1).cpu().tolist())
            labels_out.extend(labels.cpu().tolist())
            ids.extend(batch["uid"].cpu().tolist() if "uid" in batch else [])
    if was_training:
        model.train()
    counts = torch.tensor([correct, total], dtype=torch.int64, device=device if torch.device(device).type != "cpu" else "cpu")
    group = _dp_group()
    if group is not None:
        dist.all_reduce(counts, group=group)
    correct, total = int(counts[0]), int(counts[1])
    if output_predictions:
        return correct, total, (softmaxes, labels_out, ids)
    return correct, total


def accuracy_func_provider(single_dataset_provider: Callable, datapaths: Sequence, *, micro_batch_size: int,
                           device="cpu", num_workers: int = 0, log: Callable = print) -> Callable:
    """``single_dataset_provider(path)`` builds one validation set (with a ``dataset_name`` attribute); the returned
    ``metrics_func(model, epoch, output_predictions=False)`` prints the accuracy per set and overall and returns it."""
    from .finetune_utils import build_data_loader
    loaders = []
    for path in datapaths:
        ds = single_dataset_provider(path)
        loaders.append((getattr(ds, "dataset_name", str(path)),
                        build_data_loader(ds, micro_batch_size, num_workers, drop_last=False, shuffle=False)))

    def metrics_func(model, epoch, output_predictions: bool = False) -> Dict[str, float]:
        log(f"calculating metrics ... (epoch {epoch})")
        correct = total = 0
        out: Dict[str, float] = {}
        named = {}
        for name, loader in loaders:
            res = calculate_correct_answers(name, model, loader, device, output_predictions)
            c, t = res[0], res[1]
            if output_predictions:
                named[name] = res[2]
            correct += c
            total += t
            out[name] = 100.0 * c / max(t, 1)
            log(f" > |epoch: {epoch}| metrics for {name}: correct / total = {c} / {t} = {out[name]:.4f} %")
        out["overall"] = 100.0 * correct / max(total, 1)
        log(f" >> |epoch: {epoch}| overall: correct / total = {correct} / {total} = {out['overall']:.4f} %")
        if output_predictions:
            out["predictions"] = named
        return out
    return metrics_func
