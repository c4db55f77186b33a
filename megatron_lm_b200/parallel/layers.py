"""Tensor-parallel linear layers and the vocab-parallel embedding.

Behaviour follows megatron/core/tensor_parallel/layers.py (VocabParallelEmbedding
:189, ColumnParallelLinear :736, RowParallelLinear :1061): the column-parallel layer
splits the output dim, the row-parallel layer the input dim; with sequence
parallelism the column layer all-gathers its sequence-sharded input and the row
layer reduce-scatters its output, and backward mirrors this while the weight
gradient is accumulated into ``main_grad``.

One autograd function (:class:`_TPLinear`) covers every combination.  With
``tp_comm_overlap`` the gather->GEMM and GEMM->reduce-scatter pairs run as the
fused peer-memory kernels of ``ops/tp_fused.py``; otherwise the collectives are
NCCL calls issued asynchronously around the tcgen05 GEMMs.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import state
from .mappings import (_rank, _size, gather_first, reduce_scatter_first,
                       reduce_from_tensor_model_parallel_region,
                       reduce_scatter_to_sequence_parallel_region)
from .random import get_cuda_rng_tracker
from ..ops import core as ops
from ..ops.gemm import _as2d, gemm, weight_grad
from ..ops.grad import deliver
from ..ops.core import column_sum


def set_tensor_model_parallel_attributes(t: torch.Tensor, is_parallel: bool, dim: int, stride: int = 1) -> None:
    t.tensor_model_parallel = is_parallel
    t.partition_dim = dim
    t.partition_stride = stride


def _device(config):
    if config.use_cpu_initialization or not torch.cuda.is_available():
        return torch.device("cpu")
    return torch.device("cuda", torch.cuda.current_device())


def _init_sharded(weight: torch.Tensor, full_shape, partition_dim: int, init_method: Callable, config,
                  rank: int, world: int, stride: int = 1, is_expert: bool = False) -> None:
    """Initialise a TP shard.  CPU initialisation draws the full fp32 matrix from the default
    stream and slices it (so results do not depend on the TP size); device initialisation
    draws the shard under the TP (or expert) stream (reference: layers.py:128-187)."""
    if not config.perform_initialization:
        return
    if config.use_cpu_initialization or not weight.is_cuda:
        master = torch.empty(*full_shape, dtype=torch.float32)
        init_method(master)
        per = full_shape[partition_dim] // world
        if stride == 1:
            shard = master.narrow(partition_dim, rank * per, per)
        else:
            per_stride = per // stride
            pieces = torch.split(master, per_stride, dim=partition_dim)
            shard = torch.cat(pieces[rank::world], dim=partition_dim)
        with torch.no_grad():
            weight.copy_(shard.to(weight.dtype))
        return
    tracker = get_cuda_rng_tracker()
    if tracker.is_initialized():
        name = "expert-parallel-rng" if is_expert else "model-parallel-rng"
        with tracker.fork(name):
            init_method(weight)
    else:
        init_method(weight)


# Weight gradients whose GEMM was put off (``weight.defer_wgrad``): (weight, dy [tokens, N], input [tokens, K]).
# The output layer of the last pipeline stage uses this with ``defer_embedding_wgrad_compute``: its data gradient
# goes upstream at once, the large vocabulary-sized weight-gradient product runs when the pipeline drains
# (reference: megatron/core/utils.py drain_embedding_wgrad_compute, tensor_parallel/layers.py:480-500).
_DEFERRED_WGRADS: list = []


def _defer_or_compute_wgrad(weight, dy2, t2):
    if getattr(weight, "defer_wgrad", False):
        _DEFERRED_WGRADS.append((weight, dy2.detach(), t2.detach()))
        return None
    if t2.is_cuda:
        return weight_grad(weight, dy2, t2)
    return deliver(weight, dy2.float().t() @ t2.float())


def drain_deferred_wgrads(keep: int = 0, only=None) -> int:
    """Run the postponed weight-gradient products, oldest first, until at most ``keep`` remain (``only``: a set of
    ``id(weight)`` - run just the products of those weights, e.g. one layer's).  The result lands in the parameter's
    gradient buffer (or is added to ``.grad`` when there is none).  Returns how many ran."""
    ran = 0
    if only is not None:
        mine = [e for e in _DEFERRED_WGRADS if id(e[0]) in only]
        _DEFERRED_WGRADS[:] = [e for e in _DEFERRED_WGRADS if id(e[0]) not in only]
        todo = mine
    else:
        todo = None
    while (todo if todo is not None else len(_DEFERRED_WGRADS) > keep):
        weight, dy2, t2 = todo.pop(0) if todo is not None else _DEFERRED_WGRADS.pop(0)
        with torch.no_grad():
            g = weight_grad(weight, dy2, t2) if t2.is_cuda else deliver(weight, dy2.float().t() @ t2.float())
        if g is not None:
            weight.grad = g if weight.grad is None else weight.grad + g
        ran += 1
    return ran


class _TPLinear(torch.autograd.Function):
    """y = f(x) W^T with optional input all-gather (sequence parallel), output
    reduce-scatter / all-reduce, and all-reduce of the data gradient.

    With a ``fused`` communicator (CUDA, sequence parallel) the gather and the reduce-scatter
    happen inside the GEMM kernels and the gathered operand is kept for the weight gradient."""

    @staticmethod
    def forward(ctx, x, weight, bias, group, gather_input, reduce_output, allreduce_dgrad, fused):
        ctx.cfg = (group, gather_input, reduce_output, allreduce_dgrad, fused)
        ctx.bias = bias
        ctx.x_shape = x.shape
        n = _size(group)
        N = weight.shape[0]
        use_fused = fused is not None and x.is_cuda and n > 1
        ctx.use_fused = use_fused
        saved_input = x

        def product(inp, lead):
            # the result is allocated in its final shape so that the Function returns no view
            if inp.is_cuda:
                out = torch.empty(*lead, N, dtype=inp.dtype, device=inp.device)
                gemm(_as2d(inp), weight, bias=bias, out=out.view(-1, N))
                return out
            return torch.nn.functional.linear(inp, weight, bias)

        if gather_input and n > 1:
            lead = (x.shape[0] * n,) + tuple(x.shape[1:-1])
            if use_fused:
                y2, gathered = fused.ag_gemm(x, weight, bias)
                y = y2.view(*lead, N)
                saved_input = gathered            # [tp*rows, K]: kept for the weight gradient
            else:
                y = product(gather_first(x, group), lead)
        elif n > 1 and reduce_output == "reduce_scatter" and use_fused:
            lead = (x.shape[0] // n,) + tuple(x.shape[1:-1])
            y = fused.gemm_rs(x, weight).view(*lead, N)
        else:
            y = product(x, tuple(x.shape[:-1]))
            if n > 1 and reduce_output == "reduce_scatter":
                y = reduce_scatter_first(y, group)
            elif n > 1 and reduce_output == "all_reduce":
                dist.all_reduce(y, group=group)
        ctx.save_for_backward(saved_input, weight)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        group, gather_input, reduce_output, allreduce_dgrad, fused = ctx.cfg
        n = _size(group)
        if ctx.use_fused and (gather_input or reduce_output == "reduce_scatter"):
            return _TPLinear._backward_fused(ctx, dy, x, weight)
        handle = None
        total = x
        if gather_input and n > 1:
            # re-gather the sequence-sharded input while the data gradient is computed
            total = torch.empty((x.shape[0] * n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            handle = dist.all_gather_into_tensor(total, x.contiguous(), group=group, async_op=True)
        if n > 1 and reduce_output == "reduce_scatter":
            dy = gather_first(dy, group)
        dy2 = _as2d(dy) if dy.is_cuda else dy.reshape(-1, dy.shape[-1])
        dx = None
        if ctx.needs_input_grad[0]:
            if dy.is_cuda:
                dx = gemm(dy2, weight, b_mn=True)
            else:
                dx = dy2 @ weight
            dx = dx.view(*total.shape[:-1], weight.shape[1]) if handle is None else dx
        if handle is not None:
            handle.wait()
            handle = None
        rs_handle = None
        if dx is not None and n > 1:
            if gather_input:
                dx = dx.view(*total.shape)
                out = torch.empty(x.shape, dtype=dx.dtype, device=dx.device)
                rs_handle = dist.reduce_scatter_tensor(out, dx.contiguous(), group=group, async_op=True)
                dx_final = out
            elif allreduce_dgrad:
                rs_handle = dist.all_reduce(dx, group=group, async_op=True)
                dx_final = dx
            else:
                dx_final = dx
        else:
            dx_final = dx
        gw = None
        if weight.requires_grad:
            t2 = _as2d(total) if total.is_cuda else total.reshape(-1, total.shape[-1])
            gw = _defer_or_compute_wgrad(weight, dy2, t2)
        gb = None
        if ctx.bias is not None and ctx.bias.requires_grad:
            gb = deliver(ctx.bias, column_sum(dy2))
        if rs_handle is not None:
            rs_handle.wait()
        if dx_final is not None and dx_final.shape != ctx.x_shape:
            dx_final = dx_final.view(ctx.x_shape)
        return dx_final, gw, gb, None, None, None, None, None

    @staticmethod
    def _backward_fused(ctx, dy, saved, weight):
        group, gather_input, reduce_output, allreduce_dgrad, fused = ctx.cfg
        dx = gw = gb = None
        if gather_input:
            # column-parallel: dx = reduce_scatter(dy W), dW = dy^T gathered_x
            dy2 = _as2d(dy)
            if ctx.needs_input_grad[0]:
                dx = fused.gemm_rs(dy2, weight, b_mn=True).view(ctx.x_shape)
            if weight.requires_grad:
                gw = _defer_or_compute_wgrad(weight, dy2, saved)
            if ctx.bias is not None and ctx.bias.requires_grad:
                gb = deliver(ctx.bias, column_sum(dy2))
        else:
            # row-parallel: the gathered dy feeds both dx = gather(dy) W and dW = gather(dy)^T x
            x2 = _as2d(saved)
            if ctx.needs_input_grad[0]:
                dx2, dy_total = fused.ag_gemm(dy, weight, None, b_mn=True)
                dx = dx2.view(ctx.x_shape)
            else:
                dy_total = gather_first(dy, group).reshape(-1, dy.shape[-1])
            if weight.requires_grad:
                gw = weight_grad(weight, dy_total, x2)
        return dx, gw, gb, None, None, None, None, None


def tp_linear(x, weight, bias=None, *, group=None, gather_input=False, reduce_output="none",
              allreduce_dgrad=False, fused=None):
    return _TPLinear.apply(x, weight, bias, group, gather_input, reduce_output, allreduce_dgrad, fused)


def _fp8_format(module, x, w) -> Optional[str]:
    """'e4m3' / 'hybrid' when this call should run its GEMMs in FP8, else None.  FP8 applies to the linears
    of transformer layers (``fp8_eligible``), with sizes the 8-bit tensor-core path accepts (multiples of 16);
    the collectives then run outside the GEMM (the fused peer-memory kernels are 16-bit)."""
    fmt = getattr(module.config, "fp8", None)
    if not fmt or not getattr(module, "fp8_eligible", True) or x.dtype not in (torch.bfloat16, torch.float16):
        return None
    tokens = x.numel() // x.shape[-1]
    need = 32 if getattr(module.config, "fp8_recipe", None) == "mxfp8" else 16
    if tokens % need or w.shape[0] % need or w.shape[1] % need:
        return None
    return "hybrid" if fmt == "hybrid" else "e4m3"


def _fp8_linear(module):
    """The FP8 linear of the configured recipe: block-scaled MXFP8 (1 x 32 blocks, power-of-two scales in the
    tensor core) or per-tensor current scaling."""
    from ..ops.fp8 import linear_fp8, linear_mxfp8
    return linear_mxfp8 if getattr(module.config, "fp8_recipe", None) == "mxfp8" else linear_fp8


class ColumnParallelLinear(nn.Module):
    """Y = X A^T + b with A split along its output dim: A = [A_1; ...; A_p]."""

    def __init__(self, input_size: int, output_size: int, *, config, init_method: Callable, bias: bool = True,
                 gather_output: bool = False, stride: int = 1, skip_bias_add: bool = False,
                 is_expert: bool = False, tp_group=None, skip_weight_param_allocation: bool = False,
                 disable_sp_gather: bool = False):
        super().__init__()
        self.config = config
        self.input_size, self.output_size = input_size, output_size
        self.gather_output, self.skip_bias_add, self.is_expert = gather_output, skip_bias_add, is_expert
        self.tp_group = tp_group if tp_group is not None else (
            (state.get_expert_tensor_parallel_group() if is_expert else state.get_tensor_model_parallel_group())
            if state.model_parallel_is_initialized() else None)
        if state.model_parallel_is_initialized():
            world = state.get_expert_tensor_parallel_world_size() if is_expert else state.get_tensor_model_parallel_world_size()
            rank = state.get_expert_tensor_parallel_rank() if is_expert else state.get_tensor_model_parallel_rank()
        else:
            world, rank = 1, 0
        self.tp_size, self.tp_rank = world, rank
        if output_size % world:
            raise ValueError(f"output_size {output_size} not divisible by TP size {world}")
        self.output_size_per_partition = output_size // world
        self.sequence_parallel = config.sequence_parallel and world > 1 and not disable_sp_gather
        dev = _device(config)
        if not skip_weight_param_allocation:
            self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, input_size, device=dev,
                                                   dtype=config.params_dtype))
            _init_sharded(self.weight, (output_size, input_size), 0, init_method, config, rank, world, stride,
                          is_expert)
            set_tensor_model_parallel_attributes(self.weight, True, 0, stride)
            self.weight.allreduce = not (is_expert and config.expert_model_parallel_size > 1)
        else:
            self.weight = None
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, device=dev, dtype=config.params_dtype))
            set_tensor_model_parallel_attributes(self.bias, True, 0, stride)
            self.bias.allreduce = not (is_expert and config.expert_model_parallel_size > 1)
        else:
            self.register_parameter("bias", None)
        self.fused = None    # set by the model builder when tp_comm_overlap is on
        self.ptq = False     # post-training quantisation attached (post_training/ptq.py)

    def forward(self, x, weight: Optional[torch.Tensor] = None):
        w = self.weight if weight is None else weight
        b = self.bias if not self.skip_bias_add else None
        pre = False
        if self.ptq:
            from ..post_training.ptq import apply_quantizers, prequantized_linear
            x, w = apply_quantizers(self, x, w)
            pre = getattr(w, "prequantized", False)      # compressed weight fed to the FP8 GEMM as stored
        fmt = "prequant" if pre else _fp8_format(self, x, w)
        if fmt is not None:
            linear_fp8 = prequantized_linear if pre else _fp8_linear(self)
            from .mappings import copy_to_tensor_model_parallel_region, gather_from_sequence_parallel_region
            if self.sequence_parallel:
                inp = gather_from_sequence_parallel_region(x, True, self.tp_group)
            elif self.tp_size > 1:
                inp = copy_to_tensor_model_parallel_region(x, self.tp_group)
            else:
                inp = x
            y = linear_fp8(inp, w, b, fmt)
        else:
            y = tp_linear(x, w, b, group=self.tp_group, gather_input=self.sequence_parallel,
                          allreduce_dgrad=(self.tp_size > 1 and not self.sequence_parallel), fused=self.fused)
        if self.gather_output and self.tp_size > 1:
            from .mappings import gather_from_tensor_model_parallel_region
            y = gather_from_tensor_model_parallel_region(y, self.tp_group)
        return y, (self.bias if self.skip_bias_add else None)


class RowParallelLinear(nn.Module):
    """Y = X A^T + b with A split along its input dim and X split along its last dim."""

    def __init__(self, input_size: int, output_size: int, *, config, init_method: Callable, bias: bool = True,
                 input_is_parallel: bool = True, skip_bias_add: bool = False, stride: int = 1,
                 is_expert: bool = False, tp_group=None):
        super().__init__()
        self.config = config
        self.input_size, self.output_size = input_size, output_size
        self.input_is_parallel, self.skip_bias_add, self.is_expert = input_is_parallel, skip_bias_add, is_expert
        self.tp_group = tp_group if tp_group is not None else (
            (state.get_expert_tensor_parallel_group() if is_expert else state.get_tensor_model_parallel_group())
            if state.model_parallel_is_initialized() else None)
        if state.model_parallel_is_initialized():
            world = state.get_expert_tensor_parallel_world_size() if is_expert else state.get_tensor_model_parallel_world_size()
            rank = state.get_expert_tensor_parallel_rank() if is_expert else state.get_tensor_model_parallel_rank()
        else:
            world, rank = 1, 0
        self.tp_size, self.tp_rank = world, rank
        if input_size % world:
            raise ValueError(f"input_size {input_size} not divisible by TP size {world}")
        self.input_size_per_partition = input_size // world
        self.sequence_parallel = config.sequence_parallel and world > 1
        if self.sequence_parallel and not input_is_parallel:
            raise RuntimeError("sequence parallelism needs input_is_parallel=True")
        dev = _device(config)
        self.weight = nn.Parameter(torch.empty(output_size, self.input_size_per_partition, device=dev,
                                               dtype=config.params_dtype))
        _init_sharded(self.weight, (output_size, input_size), 1, init_method, config, rank, world, stride, is_expert)
        set_tensor_model_parallel_attributes(self.weight, True, 1, stride)
        self.weight.allreduce = not (is_expert and config.expert_model_parallel_size > 1)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, device=dev, dtype=config.params_dtype))
            self.bias.allreduce = not (is_expert and config.expert_model_parallel_size > 1)
            self.bias.sequence_parallel = self.sequence_parallel
        else:
            self.register_parameter("bias", None)
        self.fused = None
        self.ptq = False

    def forward(self, x):
        if not self.input_is_parallel and self.tp_size > 1:
            from .mappings import scatter_to_tensor_model_parallel_region
            x = scatter_to_tensor_model_parallel_region(x, self.tp_group)
        red = "none" if self.tp_size == 1 else ("reduce_scatter" if self.sequence_parallel else "all_reduce")
        w = self.weight
        pre = False
        if self.ptq:
            from ..post_training.ptq import apply_quantizers, prequantized_linear
            x, w = apply_quantizers(self, x, w)
            pre = getattr(w, "prequantized", False)
        fmt = "prequant" if pre else _fp8_format(self, x, w)
        if fmt is not None:
            linear_fp8 = prequantized_linear if pre else _fp8_linear(self)
            from .mappings import reduce_from_tensor_model_parallel_region, reduce_scatter_to_sequence_parallel_region
            y = linear_fp8(x, w, None, fmt)
            if red == "reduce_scatter":
                y = reduce_scatter_to_sequence_parallel_region(y, self.tp_group)
            elif red == "all_reduce":
                y = reduce_from_tensor_model_parallel_region(y, self.tp_group)
        else:
            y = tp_linear(x, w, None, group=self.tp_group, reduce_output=red, fused=self.fused)
        if self.skip_bias_add or self.bias is None:
            return y, self.bias
        return y + self.bias, None


class VocabParallelEmbedding(nn.Module):
    """Embedding table split along the vocabulary (reference: layers.py:189-314)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, init_method: Callable, config,
                 reduce_scatter_embeddings: bool = False, tp_group=None):
        super().__init__()
        self.config = config
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.reduce_scatter_embeddings = reduce_scatter_embeddings
        self.tp_group = tp_group if tp_group is not None else (
            state.get_tensor_model_parallel_group() if state.model_parallel_is_initialized() else None)
        world = state.get_tensor_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
        rank = state.get_tensor_model_parallel_rank() if state.model_parallel_is_initialized() else 0
        self.tp_size = world
        if num_embeddings % world:
            raise ValueError("vocab size must be divisible by the TP size (pad it first)")
        per = num_embeddings // world
        self.vocab_start_index, self.vocab_end_index = rank * per, (rank + 1) * per
        self.num_embeddings_per_partition = per
        self.weight = nn.Parameter(torch.empty(per, embedding_dim, device=_device(config), dtype=config.params_dtype))
        _init_sharded(self.weight, (num_embeddings, embedding_dim), 0, init_method, config, rank, world)
        set_tensor_model_parallel_attributes(self.weight, True, 0, 1)

    def forward(self, input_ids):
        out = ops.embedding(input_ids, self.weight, self.vocab_start_index, self.vocab_end_index)
        if self.tp_size == 1:
            return out
        if self.reduce_scatter_embeddings:
            out = out.transpose(0, 1).contiguous()           # [s, b, h] so the scatter is along sequence
            return reduce_scatter_to_sequence_parallel_region(out, self.tp_group)
        return reduce_from_tensor_model_parallel_region(out, self.tp_group)


def linear_with_frozen_weight(x, weight, bias=None):
    """Linear whose weight takes no gradient (reference: layers.py:317)."""
    w = weight.detach()
    return tp_linear(x, w, bias)


class LinearWithFrozenWeight:
    """Call-compatible name of the reference's autograd function (layers.py:317): ``LinearWithFrozenWeight.apply(x,
    weight, bias, allreduce_dgrad)`` - the weight receives no gradient, the data gradient is all-reduced over the
    tensor-parallel group when asked."""

    @staticmethod
    def apply(x, weight, bias=None, allreduce_dgrad: bool = False, group=None):
        w = weight.detach()
        if allreduce_dgrad:
            group = group if group is not None else (state.get_tensor_model_parallel_group()
                                                     if state.model_parallel_is_initialized() else None)
            return tp_linear(x, w, bias, group=group, allreduce_dgrad=True)
        return tp_linear(x, w, bias)
