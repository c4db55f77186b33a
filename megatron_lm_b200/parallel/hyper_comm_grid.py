"""N-dimensional communication grid with on-demand process groups (reference:
megatron/core/hyper_comm_grid.py:33-239).  ``shape`` and ``dim_names`` describe the grid, first
dimension fastest; ``create_pg("tp-dp")`` creates (collectively) the groups spanning those
dimensions and returns the one containing this rank; ``get_pg`` looks it up later."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch.distributed as dist


class HyperCommGrid:
    def __init__(self, shape: Sequence[int], dim_names: Sequence[str], rank_offset: int = 0, backend: Optional[str] = None):
        if len(shape) != len(dim_names):
            raise ValueError("shape and dim_names must have the same length")
        self.shape, self.dim_names = list(shape), list(dim_names)
        self.rank_offset, self.backend = rank_offset, backend
        self.size = int(np.prod(shape))
        if dist.is_initialized() and self.size > dist.get_world_size() - rank_offset:
            raise RuntimeError(f"grid of {self.size} ranks does not fit the world")
        self._pgs: Dict[str, object] = {}

    def _order_dims(self, dims: Union[str, Sequence[str]]):
        if isinstance(dims, str):
            dims = dims.split("-")
        for d in dims:
            if d not in self.dim_names:
                raise KeyError(f"unknown grid dimension {d}")
        ordered = [d for d in self.dim_names if d in dims]
        return ordered, "-".join(ordered)

    def _gen_rank_enum(self, dims: List[str]) -> List[List[int]]:
        grid = (np.arange(self.size) + self.rank_offset).reshape(list(reversed(self.shape)))
        axis = {n: len(self.dim_names) - 1 - i for i, n in enumerate(self.dim_names)}
        rest = [d for d in self.dim_names if d not in dims]
        perm = [axis[d] for d in reversed(rest)] + [axis[d] for d in reversed(dims)]
        gsize = int(np.prod([self.shape[self.dim_names.index(d)] for d in dims]))
        return np.transpose(grid, perm).reshape(-1, gsize).tolist()

    def create_pg(self, dims: Union[str, Sequence[str]], **kwargs):
        ordered, key = self._order_dims(dims)
        if key in self._pgs:
            raise KeyError(f"process group for {key} already exists")
        mine = None
        rank = dist.get_rank() if dist.is_initialized() else 0
        for ranks in self._gen_rank_enum(ordered):
            pg = dist.new_group(ranks, backend=self.backend, **kwargs) if dist.is_initialized() else tuple(ranks)
            if rank in ranks:
                mine = pg
        self._pgs[key] = mine
        return mine

    def get_pg(self, dims: Union[str, Sequence[str]]):
        _, key = self._order_dims(dims)
        if key not in self._pgs:
            raise KeyError(f"process group for {key} has not been created")
        return self._pgs[key]

    def get_rank_enum(self, dims: Union[str, Sequence[str]]) -> List[List[int]]:
        ordered, _ = self._order_dims(dims)
        return self._gen_rank_enum(ordered)
