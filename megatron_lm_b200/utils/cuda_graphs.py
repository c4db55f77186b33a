"""CUDA-graph capture of launch-bound pieces of the step.

Reference: megatron/core/transformer/cuda_graphs.py (``_CudaGraphRunner`` :474, ``CudaGraphManager``
:946, ``create_cudagraphs`` :323) and megatron/training/full_cuda_graph.py (``FullCudaGraphWrapper`` :97).

``GraphedModule`` captures one module's forward and backward as two graphs over static input / output
buffers and replays them from an autograd Function.  The ops of this package deliver weight gradients
by writing ``param.main_grad`` inside the kernels, so those writes are part of the backward graph; the
Python-side readiness signals that the data-parallel buckets wait for are re-issued after each replay.
``FullIterationGraph`` captures a whole forward-backward callable the same way.

Limits: no autograd graph that involves the module's parameters may be alive when the capture starts
(gradient-accumulation nodes created on another stream make the captured backward depend on uncaptured
work); shapes and tensor addresses are frozen at capture; host-chosen scalars (dropout seeds, loss
scale read on the host) are frozen too, so capture with dropout 0 or device-side RNG only.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.nn as nn

from ..ops.grad import notify_ready


def _is_cuda(ts):
    return all((not torch.is_tensor(t)) or t.is_cuda for t in ts)


class GraphedModule(nn.Module):
    def __init__(self, module: nn.Module, num_warmup: int = 3, pool=None):
        super().__init__()
        self.module = module
        self.num_warmup = num_warmup
        self.pool = pool
        self._captured = False
        self._calls = 0
        self._n_rot = 0

    def _call(self, flat):
        """The wrapped module on the flat tensor list: positional inputs, then (cos, sin) when the call came with a
        ``rotary`` pair."""
        if self._n_rot:
            return self.module(*flat[:-2], rotary=(flat[-2], flat[-1]))
        return self.module(*flat)

    # -- capture --------------------------------------------------------------------
    def _capture(self, args):
        mod = self
        params = [p for p in self.module.parameters() if p.requires_grad]
        self.params = params
        self.static_in = [a.detach().clone().requires_grad_(a.requires_grad) if torch.is_tensor(a) else a for a in args]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.num_warmup):
                out = mod._call(self.static_in)
                outs = out if isinstance(out, (tuple, list)) else (out,)
                outs_t = [o for o in outs if torch.is_tensor(o) and o.requires_grad]
                gin = [a for a in self.static_in if torch.is_tensor(a) and a.requires_grad]
                grads = torch.autograd.grad(outs_t, gin + params, [torch.ones_like(o) for o in outs_t],
                                            allow_unused=True)
                del grads
        torch.cuda.current_stream().wait_stream(side)
        for p in params:                       # warm-up passes accumulated into main_grad: undo
            if getattr(p, "main_grad", None) is not None:
                p.main_grad.zero_()
        self.fwd_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.fwd_graph, pool=self.pool):
            out = mod._call(self.static_in)
        self.out_is_tuple = isinstance(out, (tuple, list))
        outs = list(out) if self.out_is_tuple else [out]
        self.static_out = outs
        self.out_grad_idx = [i for i, o in enumerate(outs) if torch.is_tensor(o) and o.requires_grad]
        self.static_gout = [torch.zeros_like(outs[i]) for i in self.out_grad_idx]
        self.in_grad_idx = [i for i, a in enumerate(self.static_in) if torch.is_tensor(a) and a.requires_grad]
        self.bwd_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.bwd_graph, pool=self.fwd_graph.pool()):
            grads = torch.autograd.grad([outs[i] for i in self.out_grad_idx],
                                        [self.static_in[i] for i in self.in_grad_idx] + params, self.static_gout,
                                        allow_unused=True)
            n_in = len(self.in_grad_idx)
            self.static_gin = list(grads[:n_in])
            for p, g in zip(params, grads[n_in:]):            # gradients that came back through plain autograd
                if g is not None and getattr(p, "main_grad", None) is not None:
                    p.main_grad.add_(g.to(p.main_grad.dtype))
        self._captured = True

    # -- replay ----------------------------------------------------------------------
    def forward(self, *args, rotary=None, **kwargs):
        """Positional tensors and an optional ``rotary=(cos, sin)`` pair are graph inputs; any other argument that is
        not None (masks, inference contexts, encoder outputs) sends the call down the eager path."""
        if any(v is not None for v in kwargs.values()):
            return self.module(*args, rotary=rotary, **kwargs)
        n_rot = 0 if rotary is None else 2
        if self._captured and n_rot != self._n_rot:
            return self.module(*args, rotary=rotary)
        args = tuple(args) + (tuple(rotary) if rotary is not None else ())
        if not _is_cuda(args) or not torch.is_grad_enabled() and not self._captured:
            return self.module(*args[:len(args) - n_rot], rotary=rotary) if n_rot else self.module(*args)
        if not self._captured:
            self._n_rot = n_rot
            self._capture(args)
        runner = self

        class _Replay(torch.autograd.Function):
            @staticmethod
            def forward(ctx, *flat):
                for s, a in zip(runner.static_in, flat[: len(runner.static_in)]):
                    if torch.is_tensor(s):
                        s.data.copy_(a)
                runner.fwd_graph.replay()
                outs = [o.detach() if torch.is_tensor(o) else o for o in runner.static_out]
                ctx.mark_non_differentiable(*[o for i, o in enumerate(outs)
                                              if torch.is_tensor(o) and i not in runner.out_grad_idx])
                return tuple(outs)

            @staticmethod
            def backward(ctx, *gouts):
                for s, i in zip(runner.static_gout, runner.out_grad_idx):
                    s.copy_(gouts[i])
                runner.bwd_graph.replay()
                for p in runner.params:
                    if getattr(p, "main_grad", None) is not None:
                        notify_ready(p)
                res: List[Optional[torch.Tensor]] = [None] * len(runner.static_in)
                for g, i in zip(runner.static_gin, runner.in_grad_idx):
                    res[i] = None if g is None else g.detach().clone()
                return tuple(res) + (None,) * len(runner.params)

        tensors = [a if torch.is_tensor(a) else torch.empty(0) for a in args]
        outs = _Replay.apply(*tensors, *self.params)
        return outs if self.out_is_tuple else outs[0]


def _graphed_getattr(self, name):
    try:
        return nn.Module.__getattr__(self, name)
    except AttributeError:
        mod = self.__dict__.get("_modules", {}).get("module")
        if mod is None:
            raise
        return getattr(mod, name)


GraphedModule.__getattr__ = _graphed_getattr          # layer_number, self_attention, ... of the wrapped layer


class CudaGraphManager:
    """Wraps selected sub-modules (by default every transformer layer) of a model in ``GraphedModule``."""

    def __init__(self, model: nn.Module, layer_types: Optional[Sequence[type]] = None, num_warmup: int = 3):
        if layer_types is None:
            from ..models.transformer import TransformerLayer
            layer_types = (TransformerLayer,)
        self.wrapped = []
        pool = torch.cuda.graph_pool_handle() if torch.cuda.is_available() else None
        for name, parent in list(model.named_modules()):
            for child_name, child in list(parent.named_children()):
                if isinstance(child, tuple(layer_types)):
                    g = GraphedModule(child, num_warmup, pool)
                    setattr(parent, child_name, g)
                    self.wrapped.append(g)


class FullIterationGraph:
    """Capture ``fn(*static_tensors)`` (e.g. all microbatches' forward+backward) once and replay it with new
    data copied into the static tensors.  ``fn`` must not synchronise with the host."""

    def __init__(self, fn: Callable, num_warmup: int = 2):
        self.fn, self.num_warmup = fn, num_warmup
        self.graph = None

    def __call__(self, *tensors):
        if not _is_cuda(tensors):
            return self.fn(*tensors)
        if self.graph is None:
            self.static = [t.clone() for t in tensors]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(self.num_warmup):
                    self.fn(*self.static)
            torch.cuda.current_stream().wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.result = self.fn(*self.static)
        else:
            for s, t in zip(self.static, tensors):
                s.copy_(t)
        self.graph.replay()
        return self.result
