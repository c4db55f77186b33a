"""Small library utilities shared across the package.

Reference: megatron/core/utils.py - ``check_param_hashes_across_dp_replicas`` :685, NVTX helpers
:1874-1965, ``unwrap_model`` :1995, ``make_viewless_tensor`` :584, ``get_model_config``, divide/ceil helpers.
"""
from __future__ import annotations

import functools
import hashlib
from contextlib import contextmanager
from typing import Iterable, List, Optional, Sequence

import torch
import torch.distributed as dist

_NVTX_ENABLED = False


def configure_nvtx_profiling(enabled: bool) -> None:
    global _NVTX_ENABLED
    _NVTX_ENABLED = bool(enabled)


def nvtx_range_push(msg: Optional[str] = None, suffix: Optional[str] = None) -> None:
    if _NVTX_ENABLED and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(f"{msg or 'range'}{'.' + suffix if suffix else ''}")


def nvtx_range_pop(msg: Optional[str] = None, suffix: Optional[str] = None) -> None:
    if _NVTX_ENABLED and torch.cuda.is_available():
        torch.cuda.nvtx.range_pop()


@contextmanager
def nvtx_range(msg: str):
    nvtx_range_push(msg)
    try:
        yield
    finally:
        nvtx_range_pop(msg)


def nvtx_decorator(message: Optional[str] = None):
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*a, **kw):
            nvtx_range_push(message or fn.__qualname__)
            try:
                return fn(*a, **kw)
            finally:
                nvtx_range_pop()
        return wrapped
    return deco


def unwrap_model(model, module_instances=None):
    """Strip wrappers that expose ``.module`` (data-parallel buffers, half-precision wrapper)."""
    as_list = isinstance(model, (list, tuple))
    out = []
    for m in (model if as_list else [model]):
        while hasattr(m, "module") and (module_instances is None or isinstance(m, module_instances)):
            m = m.module
        out.append(m)
    return out if as_list else out[0]


def make_viewless_tensor(inp: torch.Tensor, requires_grad: bool, keep_graph: bool) -> torch.Tensor:
    """A tensor sharing ``inp``'s storage that is not a view of anything (its ``_base`` is None), so that freeing
    the original's storage is not blocked by view bookkeeping."""
    if inp._base is None:
        return inp
    if keep_graph:
        return _MakeViewless.apply(inp, requires_grad)
    out = torch.empty((1,), dtype=inp.dtype, device=inp.device, requires_grad=requires_grad)
    out.data = inp.data
    return out


class _MakeViewless(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inp, requires_grad):
        out = torch.empty((1,), dtype=inp.dtype, device=inp.device, requires_grad=requires_grad)
        out.data = inp.data
        return out

    @staticmethod
    def backward(ctx, g):
        return g, None


def param_hash(t: torch.Tensor) -> str:
    return hashlib.sha1(t.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes()).hexdigest()


def check_param_hashes_across_dp_replicas(model: Sequence[torch.nn.Module], cross_check: bool = False) -> bool:
    """True when every data-parallel replica holds bit-identical parameters (and fp32 master copies when the
    parameters carry ``main_param``).  All ranks of the data-parallel group call."""
    from ..parallel import state
    local = []
    for i, chunk in enumerate(model):
        for n, p in chunk.named_parameters():
            local.append((i, n, param_hash(p.data)))
            mp = getattr(p, "main_param", None)
            if mp is not None:
                local.append((i, n + ".main", param_hash(mp)))
    if not dist.is_initialized():
        return True
    group = state.get_data_parallel_group() if state.model_parallel_is_initialized() else dist.group.WORLD
    world = dist.get_world_size(group)
    gathered: List[Optional[list]] = [None] * world
    dist.all_gather_object(gathered, local, group=group)
    ok = all(g == gathered[0] for g in gathered)
    if cross_check and not ok:
        for a, b in zip(gathered[0], gathered[-1]):
            if a != b:
                raise RuntimeError(f"parameter {a[1]} (chunk {a[0]}) differs between data-parallel replicas")
    return ok


def divide(a: int, b: int) -> int:
    if a % b:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def get_model_config(model):
    return unwrap_model(model).config


def drain_embedding_wgrad_compute(config=None, *_unused, keep: int = 0) -> int:
    """Run the output layer's postponed weight-gradient products (``defer_embedding_wgrad_compute``); the pipelined
    schedule calls this by itself, a hand-written loop calls it before the gradients are reduced
    (reference: megatron/core/utils.py drain_embedding_wgrad_compute)."""
    from ..parallel.layers import drain_deferred_wgrads
    return drain_deferred_wgrads(keep)


# ---------------------------------------------------------------------------------------------- multi-tensor fallbacks
def local_multi_tensor_applier(op, noop_flag_buffer, tensor_lists, *args):
    """Call convention of the fused multi-tensor kernels (reference: megatron/core/utils.py:1032-1051): ``op`` gets the
    chunk size (unused here), the no-op flag, the tensor lists and the extra arguments."""
    return op(2048 * 32, noop_flag_buffer, tensor_lists, *args)


def local_multi_tensor_l2_norm(chunk_size, noop_flag, tensor_lists, per_tensor: bool = False, *args):
    """L2 norm over all tensors of ``tensor_lists[0]`` as a one-element fp32 tensor (and the per-tensor norms when
    asked): ``torch._foreach_norm`` does the work in a few launches on a GPU."""
    tensors = list(tensor_lists[0])
    if not tensors:
        z = torch.zeros(1, dtype=torch.float32)
        return z, (z.clone() if per_tensor else None)
    norms = torch.stack([n.float() for n in torch._foreach_norm(tensors, 2)])
    total = torch.linalg.vector_norm(norms, 2).reshape(1)
    return total, (norms if per_tensor else None)


def local_multi_tensor_scale(chunk_size, noop_flag, tensor_lists, scale):
    """``dst[i] = src[i] * scale`` for the tensor pairs of ``tensor_lists = [srcs, dsts]``."""
    srcs, dsts = tensor_lists
    for s, d in zip(srcs, dsts):
        d.copy_(s * scale)
