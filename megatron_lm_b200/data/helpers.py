"""ctypes front-end of the C++ index builders in ``helpers.cpp`` (built in-tree with g++)."""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
from typing import Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "helpers.cpp")
_LIB = os.path.join(_HERE, "..", "_C", "libmlb_data.so")
_lib: Optional[ctypes.CDLL] = None


def build(force: bool = False) -> str:
    lib = os.path.normpath(_LIB)
    if not force and os.path.exists(lib) and os.path.getmtime(lib) > os.path.getmtime(_SRC):
        return lib
    os.makedirs(os.path.dirname(lib), exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    r = subprocess.run([cxx, "-O3", "-std=c++17", "-shared", "-fPIC", "-o", lib, _SRC], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building dataset helpers failed:\n{r.stderr}")
    return lib


def _load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.mlb_num_samples.restype = ctypes.c_int64
        _lib.mlb_num_samples.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
        _lib.mlb_build_sample_idx.restype = ctypes.c_int
        _lib.mlb_build_sample_idx.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64,
                                              ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                              ctypes.c_void_p]
        _lib.mlb_build_blending_indices.restype = None
        _lib.mlb_build_blending_indices.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                                    ctypes.c_int64]
        _lib.mlb_build_exhaustive_blending_indices.restype = None
        _lib.mlb_build_exhaustive_blending_indices.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                               ctypes.c_int32]
        _lib.mlb_build_mapping.restype = ctypes.c_int64
        _lib.mlb_build_mapping.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int32,
                                           ctypes.c_int64, ctypes.c_int32, ctypes.c_double, ctypes.c_int32,
                                           ctypes.c_int32, ctypes.c_void_p]
        _lib.mlb_build_blocks_mapping.restype = ctypes.c_int64
        _lib.mlb_build_blocks_mapping.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                                  ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                                  ctypes.c_int32, ctypes.c_void_p]
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def build_sample_idx(sizes: np.ndarray, document_idx: np.ndarray, seq_length: int, num_epochs: int,
                     tokens_per_epoch: int, drop_last_partial_sequence: bool = True,
                     add_extra_token_to_sequence: int = 1) -> np.ndarray:
    L = _load()
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    if document_idx.dtype not in (np.int32, np.int64):
        document_idx = document_idx.astype(np.int64)
    document_idx = np.ascontiguousarray(document_idx)
    n = L.mlb_num_samples(num_epochs, tokens_per_epoch, seq_length, int(add_extra_token_to_sequence),
                          int(drop_last_partial_sequence))
    out = np.zeros((n + 1, 2), dtype=np.int64)
    rc = L.mlb_build_sample_idx(_p(sizes), _p(document_idx), int(document_idx.dtype == np.int64), len(document_idx),
                                seq_length, n, int(add_extra_token_to_sequence), int(drop_last_partial_sequence),
                                _p(out))
    if rc != 0:
        raise ValueError("document index does not hold enough tokens for the requested samples")
    return out


def build_blending_indices(weights, size: int) -> Tuple[np.ndarray, np.ndarray]:
    L = _load()
    w = np.ascontiguousarray(weights, dtype=np.float64)
    di = np.zeros(size, dtype=np.int16)
    dsi = np.zeros(size, dtype=np.int64)
    L.mlb_build_blending_indices(_p(di), _p(dsi), _p(w), len(w), size)
    return di, dsi


def build_exhaustive_blending_indices(sizes) -> Tuple[np.ndarray, np.ndarray]:
    L = _load()
    s = np.ascontiguousarray(sizes, dtype=np.int64)
    total = int(s.sum())
    di = np.zeros(total, dtype=np.int16)
    dsi = np.zeros(total, dtype=np.int64)
    L.mlb_build_exhaustive_blending_indices(_p(di), _p(dsi), _p(s), len(s))
    return di, dsi


def build_mapping(docs, sizes, num_epochs: int, max_num_samples: int, max_seq_length: int, short_seq_prob: float,
                  seed: int, min_num_sent: int = 2) -> np.ndarray:
    L = _load()
    docs = np.ascontiguousarray(docs, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    args = (_p(docs), len(docs) - 1, _p(sizes), num_epochs, max_num_samples, max_seq_length, short_seq_prob, seed,
            min_num_sent)
    n = L.mlb_build_mapping(*args, None)
    out = np.zeros((n, 3), dtype=np.int64)
    L.mlb_build_mapping(*args, _p(out))
    return out


def build_blocks_mapping(docs, sizes, title_sizes, num_epochs: int, max_num_samples: int, max_seq_length: int,
                         seed: int, use_one_sent_blocks: bool = False) -> np.ndarray:
    L = _load()
    docs = np.ascontiguousarray(docs, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    title_sizes = np.ascontiguousarray(title_sizes, dtype=np.int32)
    args = (_p(docs), len(docs) - 1, _p(sizes), _p(title_sizes), num_epochs, max_num_samples, max_seq_length, seed,
            int(use_one_sent_blocks))
    n = L.mlb_build_blocks_mapping(*args, None)
    out = np.zeros((n, 4), dtype=np.int64)
    L.mlb_build_blocks_mapping(*args, _p(out))
    return out
