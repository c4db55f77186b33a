"""Epoch-based fine-tuning of classification-style models on down-stream tasks.

Reference: tasks/finetune_utils.py (``process_batch`` :26, ``cross_entropy_loss_func`` :40, ``build_data_loader`` :72
with a ``DistributedSampler`` over the data-parallel group, ``_build_infinite_size_dataloader`` :95, ``_train`` :145 -
epochs, per-epoch evaluation callback, checkpoint at the save interval and at the end - and ``finetune`` :239:
datasets -> model and optimizer -> optional pre-trained checkpoint -> train or evaluate only).
The step itself is the framework's ``train_step`` (micro-batches, gradient reduction, optimizer, scheduler), so
tensor-, pipeline- and data-parallel fine-tuning behave as in pre-training.
"""
from __future__ import annotations

import math
import time
from functools import partial
from typing import Callable, Dict, Iterable, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel import state


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


def _cross_entropy_forward_step(device, batch, model):
    """One micro-batch: ``batch`` is an iterator (the schedules pull from it) or a ready batch."""
    try:
        b = next(batch)
    except TypeError:
        b = batch
    tokens, types, labels, mask = process_batch(b, device)
    return model(tokens, mask, types), partial(cross_entropy_loss_func, labels)


@torch.no_grad()
def calculate_correct_answers(model: Callable, loader: Iterable, device) -> Dict[str, float]:
    correct = total = 0
    for batch in loader:
        tokens, types, labels, mask = process_batch(batch, device)
        logits = model(tokens, mask, types)
        correct += int((logits.argmax(-1) == labels).sum())
        total += labels.numel()
    return {"correct": correct, "total": total, "accuracy": correct / max(total, 1)}


def build_data_loader(dataset, micro_batch_size: int, num_workers: int = 0, drop_last: bool = True,
                      shuffle: bool = True, seed: int = 1234):
    """Every data-parallel rank reads its own 1/dp of the set (shuffled per epoch through ``sampler.set_epoch``)."""
    if dist.is_initialized() and state.model_parallel_is_initialized():
        world, rank = state.get_data_parallel_world_size(), state.get_data_parallel_rank()
    else:
        world, rank = 1, 0
    sampler = torch.utils.data.distributed.DistributedSampler(dataset, num_replicas=world, rank=rank, shuffle=shuffle,
                                                              seed=seed, drop_last=False)
    return torch.utils.data.DataLoader(dataset, batch_size=micro_batch_size, sampler=sampler, shuffle=False,
                                       num_workers=num_workers, drop_last=drop_last, pin_memory=torch.cuda.is_available())


def _build_infinite_size_dataloader(loader):
    """Validation during training never runs dry: start over when a pass ends."""
    it = iter(loader)
    while True:
        try:
            yield next(it)
        except StopIteration:
            it = iter(loader)


def finetune(train_valid_datasets_provider: Callable, model_provider: Callable, *, config, optimizer_config,
             epochs: int, micro_batch_size: int, global_batch_size: Optional[int] = None, lr_warmup_fraction: float = 0.0,
             lr_decay_style: str = "linear", forward_step: Optional[Callable] = None,
             end_of_epoch_callback_provider: Optional[Callable] = None, pretrained_checkpoint: Optional[str] = None,
             load_pretrained: Optional[Callable] = None, save: Optional[Callable] = None, save_interval: Optional[int] = None,
             log_interval: int = 10, seq_length: int = 0, device="cpu", num_workers: int = 0, seed: int = 1234,
             log: Callable = print) -> Dict:
    """Fine-tune for ``epochs`` passes over the training set (``epochs == 0``: evaluate only).

    ``train_valid_datasets_provider()`` -> (train set, validation set or None); ``model_provider(pre_process,
    post_process)`` -> model chunk; ``end_of_epoch_callback_provider()`` -> ``callback(model, epoch)`` (accuracy on
    the validation sets); ``load_pretrained(model_chunks, path)`` loads the pre-trained encoder; ``save(iteration,
    model_chunks, optimizer, scheduler)`` writes a checkpoint.  Returns the history."""
    from ..training.training import (build_optimizer, get_model, get_optimizer_param_scheduler, install_callbacks,
                                     train_step)
    dp = state.get_data_parallel_world_size() if state.model_parallel_is_initialized() else 1
    global_batch_size = global_batch_size or micro_batch_size * dp
    if global_batch_size % (micro_batch_size * dp):
        raise ValueError("global batch size must be a multiple of micro batch size x data-parallel size")
    num_micro = global_batch_size // (micro_batch_size * dp)
    train_ds, valid_ds = train_valid_datasets_provider() if epochs > 0 else (None, None)
    train_loader = build_data_loader(train_ds, micro_batch_size, num_workers, True, True, seed) if train_ds is not None else None
    iters_per_epoch = len(train_loader) // num_micro if train_loader is not None else 0
    train_iters = epochs * iters_per_epoch
    callback = end_of_epoch_callback_provider() if end_of_epoch_callback_provider is not None else None
    model = get_model(lambda **kw: model_provider(**{k: v for k, v in kw.items() if k in ("pre_process", "post_process")}),
                      config)
    history: Dict = {"losses": [], "metrics": [], "iterations": 0}
    if pretrained_checkpoint is not None:
        if load_pretrained is None:
            raise ValueError("pretrained_checkpoint needs a load_pretrained(model_chunks, path) function")
        load_pretrained(model, pretrained_checkpoint)
    if epochs == 0:
        if callback is not None:
            history["metrics"].append(callback(model[0], epoch=-1))
        return history
    optimizer = build_optimizer(optimizer_config, model)
    scheduler = get_optimizer_param_scheduler(
        optimizer, lr=optimizer_config.lr, min_lr=optimizer_config.min_lr, lr_decay_style=lr_decay_style,
        train_iters=max(train_iters, 1), global_batch_size=global_batch_size, lr_warmup_fraction=lr_warmup_fraction,
        weight_decay=optimizer_config.weight_decay)
    install_callbacks(config, model, optimizer)
    step_fn = forward_step or partial(_cross_entropy_forward_step, device)
    for m in model:
        m.train()
    iteration, t0, window = 0, time.time(), []
    for epoch in range(epochs):
        log(f"working on epoch {epoch + 1} ...")
        train_loader.sampler.set_epoch(seed + epoch)
        it = iter(train_loader)
        for _ in range(iters_per_epoch):
            losses, skipped, grad_norm, _ = train_step(step_fn, it, model, optimizer, scheduler, config,
                                                       num_microbatches=num_micro, seq_length=seq_length,
                                                       micro_batch_size=micro_batch_size,
                                                       global_batch_size=global_batch_size)
            iteration += 1
            if "lm loss" in losses:
                val = float(losses["lm loss"])
                if not math.isfinite(val):
                    raise FloatingPointError(f"loss is {val} at iteration {iteration}")
                window.append(val)
                history["losses"].append(val)
            if log_interval and iteration % log_interval == 0:
                lr = optimizer.param_groups[0]["lr"]
                log(f" iteration {iteration:8d}/{train_iters:8d} | epoch {epoch + 1} | "
                    f"elapsed per iteration (ms): {(time.time() - t0) * 1000 / log_interval:.1f} | learning rate: {lr:.3E} | "
                    f"lm loss: {sum(window) / max(len(window), 1):.6E} | skipped: {skipped}")
                t0, window = time.time(), []
            if save is not None and save_interval and iteration % save_interval == 0:
                save(iteration, model, optimizer, scheduler)
        if save is not None:
            save(iteration, model, optimizer, scheduler)
        if callback is not None:
            history["metrics"].append(callback(model[0], epoch=epoch))
    history["iterations"] = iteration
    history["model"] = model
    return history
