"""Dump the constructor configuration of modules as JSON files (reference:
megatron/core/config_logger.py:85): ``--config-logger-dir`` collects, per class, the arguments each
instance was built with, numbered per rank."""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict

import torch
import torch.distributed as dist

_COUNTS: Dict[str, int] = {}


def has_config_logger_enabled(config) -> bool:
    return bool(getattr(config, "config_logger_dir", ""))


def _jsonable(o: Any):
    if dataclasses.is_dataclass(o) and not isinstance(o, type):
        return {f.name: _jsonable(getattr(o, f.name)) for f in dataclasses.fields(o)}
    if isinstance(o, dict):
        return {str(k): _jsonable(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [_jsonable(v) for v in o]
    if isinstance(o, (int, float, str, bool)) or o is None:
        return o
    if isinstance(o, torch.dtype):
        return str(o)
    if callable(o):
        return getattr(o, "__name__", repr(o))
    return repr(o)


def log_config_to_disk(config, dict_data: Dict[str, Any], prefix: str = "") -> str:
    d = config.config_logger_dir
    os.makedirs(d, exist_ok=True)
    rank = dist.get_rank() if dist.is_initialized() else 0
    key = prefix or "config"
    n = _COUNTS.get(key, 0)
    _COUNTS[key] = n + 1
    path = os.path.join(d, f"{key}.rank_{rank}.iter_{n}.json")
    with open(path, "w") as f:
        json.dump(_jsonable(dict_data), f, indent=2)
    return path
