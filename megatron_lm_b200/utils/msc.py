"""Optional multi-storage client: one switch that says whether paths may be handed to the ``multistorageclient``
package (object stores behind ``msc://`` profiles) or are opened as plain files.

``MultiStorageClientFeature.is_enabled()`` is true only when the package is importable and the run did not pass
``--disable-msc``; ``open_file`` / ``path_exists`` / ``makedirs`` route through the package in that case and fall back
to the local file system otherwise.  Reference: megatron/core/msc_utils.py:21-69.
"""
from __future__ import annotations

import os
from typing import Any

try:
    import multistorageclient as _msc          # absent in most installations
except ModuleNotFoundError:                     # pragma: no cover - depends on the environment
    _msc = None


class _FeatureFlag:
    def __init__(self, default: bool = False):
        self._enabled = default

    def enable(self) -> None:
        self._enabled = True

    def disable(self) -> None:
        self._enabled = False

    def is_enabled(self) -> bool:
        return self._enabled and _msc is not None

    def import_package(self) -> Any:
        if _msc is None:
            raise RuntimeError("the multistorageclient package is not installed (pip install multi-storage-client)")
        if not self.is_enabled():
            raise RuntimeError("the multi-storage client is switched off (--disable-msc)")
        return _msc

    def __getstate__(self):
        return {"_enabled": self._enabled}

    def __setstate__(self, state):
        self._enabled = state["_enabled"]


MultiStorageClientFeature = _FeatureFlag(_msc is not None)


def configure_from_args(args) -> bool:
    """``--disable-msc`` (dest ``enable_msc``) switches the feature off for the run."""
    if getattr(args, "enable_msc", True):
        MultiStorageClientFeature.enable()
    else:
        MultiStorageClientFeature.disable()
    return MultiStorageClientFeature.is_enabled()


def open_file(path, *args, **kwargs):
    if MultiStorageClientFeature.is_enabled():
        return MultiStorageClientFeature.import_package().open(path, *args, **kwargs)
    return open(path, *args, **kwargs)


def path_exists(path) -> bool:
    if MultiStorageClientFeature.is_enabled():
        msc = MultiStorageClientFeature.import_package()
        return msc.Path(path).exists()
    return os.path.exists(path)


def makedirs(path, exist_ok: bool = True) -> None:
    if MultiStorageClientFeature.is_enabled():
        msc = MultiStorageClientFeature.import_package()
        msc.Path(path).mkdir(parents=True, exist_ok=exist_ok)
        return
    os.makedirs(path, exist_ok=exist_ok)
