"""Process-wide singletons of a training job: parsed arguments, timers, tokenizer, metric writers,
signal handler, energy monitor.

Reference: megatron/training/global_vars.py (getters :26-76, ``set_global_variables`` :84,
writer set-up :175-260) and one_logger_utils.py (callbacks are no-ops without the external package).
"""
from __future__ import annotations

import os
import time
from typing import Any, Optional

_GLOBALS = {"args": None, "timers": None, "tokenizer": None, "tensorboard": None, "wandb": None, "one_logger": None,
            "signal_handler": None, "energy_monitor": None, "adlr_autoresume": None, "num_microbatches": None}


def _need(name):
    v = _GLOBALS[name]
    if v is None:
        raise RuntimeError(f"{name} is not initialized")
    return v


def get_args(): return _need("args")
def get_timers(): return _need("timers")
def get_tokenizer(): return _need("tokenizer")
def get_tensorboard_writer(): return _GLOBALS["tensorboard"]
def get_wandb_writer(): return _GLOBALS["wandb"]
def get_one_logger(): return _GLOBALS["one_logger"]
def get_adlr_autoresume(): return _GLOBALS["adlr_autoresume"]
def get_signal_handler(): return _need("signal_handler")
def get_energy_monitor(): return _GLOBALS["energy_monitor"]


def set_args(args): _GLOBALS["args"] = args


def unset_global_variables():
    for k in _GLOBALS:
        _GLOBALS[k] = None


class _JsonlWriter:
    """Fallback metric sink with the SummaryWriter methods the loop uses: one JSON line per scalar."""

    def __init__(self, path):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.f = open(path, "a")

    def add_scalar(self, tag, value, step=None):
        import json
        self.f.write(json.dumps({"tag": tag, "value": float(value), "step": step, "time": time.time()}) + "\n")

    def add_text(self, tag, text, global_step=None):
        import json
        self.f.write(json.dumps({"tag": tag, "text": str(text), "step": global_step}) + "\n")

    def log(self, metrics: dict, step=None):
        for k, v in metrics.items():
            self.add_scalar(k, v, step)

    def flush(self): self.f.flush()
    def close(self): self.f.close()
    finish = close


class OneLoggerStub:
    """Accepts the callback surface of the one-logger integration and records the last values."""

    def __init__(self, project: str = "", run_name: str = "", app_tag_run_name: str = "", app_tag_run_version: str = "",
                 is_async: bool = False):
        """The identity of the run as the flags give it (``--one-logger-project``, ``--one-logger-run-name``,
        ``--app-tag-run-name``, ``--app-tag-run-version``, ``--one-logger-async``) goes into the record."""
        self.store = {"project": project, "run_name": run_name, "app_tag_run_name": app_tag_run_name,
                      "app_tag_run_version": app_tag_run_version, "async": bool(is_async)}

    def log_metrics(self, metrics: dict):
        self.store.update(metrics)

    def store_set(self, k, v): self.store[k] = v
    def store_get(self, k): return self.store.get(k)
    def store_has_key(self, k): return k in self.store
    def on_train_start(self, **kw): self.store.update(kw)
    def on_save_checkpoint_start(self, **kw): self.store.update(kw)
    def on_save_checkpoint_end(self, **kw): self.store.update(kw)
    def on_app_end(self, **kw): self.store.update(kw)


def _is_last_rank(args) -> bool:
    return getattr(args, "rank", 0) == getattr(args, "world_size", 1) - 1


def set_global_variables(args, build_tokenizer: bool = True):
    from ..utils.timers import Timers
    set_args(args)
    _GLOBALS["timers"] = Timers(getattr(args, "timing_log_level", 0), getattr(args, "timing_log_option", "minmax"))
    if build_tokenizer and getattr(args, "tokenizer_type", None):
        from ..data.tokenizer import build_tokenizer as _bt
        _GLOBALS["tokenizer"] = _bt(args)
    if getattr(args, "tensorboard_dir", None) and _is_last_rank(args):
        try:
            from torch.utils.tensorboard import SummaryWriter
            _GLOBALS["tensorboard"] = SummaryWriter(log_dir=args.tensorboard_dir,
                                                    max_queue=getattr(args, "tensorboard_queue_size", 1000))
        except Exception:
            _GLOBALS["tensorboard"] = _JsonlWriter(os.path.join(args.tensorboard_dir, "scalars.jsonl"))
    if getattr(args, "wandb_project", None) and _is_last_rank(args):
        try:
            import wandb
            wandb.init(dir=getattr(args, "wandb_save_dir", None) or "wandb", name=getattr(args, "wandb_exp_name", ""),
                       project=args.wandb_project, config=vars(args))
            _GLOBALS["wandb"] = wandb
        except Exception:
            _GLOBALS["wandb"] = _JsonlWriter(os.path.join(getattr(args, "wandb_save_dir", None) or "wandb",
                                                          "metrics.jsonl"))
    if getattr(args, "enable_one_logger", False) and _is_last_rank(args):
        _GLOBALS["one_logger"] = OneLoggerStub(getattr(args, "one_logger_project", "") or "",
                                               getattr(args, "one_logger_run_name", "") or "",
                                               getattr(args, "app_tag_run_name", "") or "",
                                               getattr(args, "app_tag_run_version", "") or "",
                                               getattr(args, "one_logger_async", False))
    if getattr(args, "exit_signal_handler", False):
        from .resilience import DistributedSignalHandler
        _GLOBALS["signal_handler"] = DistributedSignalHandler().__enter__()
    if getattr(args, "log_energy", False):
        from ..utils.energy_monitor import EnergyMonitor
        _GLOBALS["energy_monitor"] = EnergyMonitor()
    return args
