"""``ModuleSpec`` / ``build_module`` (reference: megatron/core/transformer/spec_utils.py:9-106).

This framework wires its transformer directly (one implementation per op), but user code written
against the reference composes custom blocks through specs, so the mechanism is kept: a spec names
a module class (or import path), constructor params and sub-module specs."""
from __future__ import annotations

import importlib
import types
from dataclasses import dataclass, field
from typing import Any, Tuple, Union


@dataclass
class ModuleSpec:
    module: Union[Tuple[str, str], type]
    params: dict = field(default_factory=dict)
    submodules: Any = None


def import_module(path: Tuple[str, str]):
    mod_path, name = path
    return getattr(importlib.import_module(mod_path), name)


def get_module(spec_or_module: Union[ModuleSpec, type], **extra):
    if isinstance(spec_or_module, ModuleSpec):
        m = spec_or_module.module
        return import_module(m) if isinstance(m, tuple) else m
    return spec_or_module


def build_module(spec_or_module: Union[ModuleSpec, type, types.FunctionType], *args, **kwargs):
    if isinstance(spec_or_module, types.FunctionType):
        return spec_or_module
    if isinstance(spec_or_module, ModuleSpec) and isinstance(spec_or_module.module, types.FunctionType):
        return spec_or_module.module
    if isinstance(spec_or_module, type):
        return spec_or_module(*args, **kwargs)
    module = get_module(spec_or_module)
    if isinstance(module, types.FunctionType):
        return module
    params = dict(spec_or_module.params)
    if spec_or_module.submodules is not None:
        kwargs["submodules"] = spec_or_module.submodules
    try:
        return module(*args, **params, **kwargs)
    except Exception as e:
        raise type(e)(f"{e} when instantiating {module.__name__}").with_traceback(e.__traceback__)
