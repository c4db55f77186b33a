"""GF(2^8) matrix application on byte buffers: ``dst_i = XOR_j M[i][j] * src_j``.

CUDA: one launch of ``csrc/ec.cu`` over up to 16 sources that may be peer-mapped addresses of
other GPUs (the parity owner pulls the stripe members over NVLink and multiplies+XORs in one pass).
CPU: table look-ups (``checkpoint/gf256.apply_matrix_numpy``), which is also the oracle."""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Union

import numpy as np
import torch

from . import _lib
from ..checkpoint import gf256

_lib.register_signatures({"mlb_ec_apply": "pppiilip"})


def ec_apply(matrix: np.ndarray, srcs: Sequence[Union[torch.Tensor, int]], dsts: Sequence[torch.Tensor], nbytes: int,
             max_blocks: int = 0) -> None:
    """``srcs`` entries are uint8-viewable CUDA tensors or raw device addresses (peer pointers)."""
    m, k = matrix.shape
    if all(torch.is_tensor(s) and not s.is_cuda for s in srcs):
        outs = gf256.apply_matrix_numpy(matrix, [s.view(torch.uint8).numpy()[:nbytes] for s in srcs])
        for d, o in zip(dsts, outs):
            d.view(torch.uint8)[:nbytes].copy_(torch.from_numpy(o))
        return
    sp = (ctypes.c_void_p * k)(*[int(s.data_ptr()) if torch.is_tensor(s) else int(s) for s in srcs])
    dp = (ctypes.c_void_p * m)(*[int(d.data_ptr()) for d in dsts])
    co = np.ascontiguousarray(matrix, dtype=np.uint8)
    _lib.check(_lib.lib().mlb_ec_apply(sp, dp, co.ctypes.data_as(ctypes.c_void_p), k, m, int(nbytes), max_blocks,
                                       _lib.stream()), "ec_apply")
