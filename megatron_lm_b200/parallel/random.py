"""Named RNG streams and activation checkpointing.

Model-parallel regions need different random streams: dropout on activations
that are replicated across the TP group must agree between ranks, dropout on
TP- or sequence-sharded activations must differ, expert-parallel ranks draw
their own initialisations.  Seeds follow the reference exactly
(megatron/core/tensor_parallel/random.py:326-377): default stream = ``seed``,
TP stream = ``seed + 2718 + tp_rank``, expert stream =
``seed + 1024 + 100 * ep_rank + etp_rank``.

The tracker stores generator *states* and swaps them into the device's default
generator inside ``fork`` - on CUDA when available, otherwise on the CPU
generator, so the same code runs in the CPU/Gloo configuration.
"""
from __future__ import annotations

import contextlib
from typing import Dict, Optional

import torch

from . import state

_MODEL_PARALLEL_RNG = "model-parallel-rng"
_DATA_PARALLEL_RNG = "data-parallel-rng"
_EXPERT_PARALLEL_RNG = "expert-parallel-rng"


def _get_state(cuda: bool):
    return torch.cuda.get_rng_state() if cuda else torch.get_rng_state()


def _set_state(s, cuda: bool):
    if cuda:
        torch.cuda.set_rng_state(s)
    else:
        torch.set_rng_state(s)


class RNGStatesTracker:
    def __init__(self):
        self.reset()

    def reset(self):
        self.states_: Dict[str, torch.Tensor] = {}
        self.seeds_ = set()
        self.cuda = torch.cuda.is_available()

    def is_initialized(self) -> bool:
        return len(self.states_) > 0

    def get_states(self):
        return {k: v.clone() for k, v in self.states_.items()}

    def set_states(self, states):
        self.states_ = {k: v.clone() for k, v in states.items()}

    def add(self, name: str, seed: int):
        if seed in self.seeds_:
            raise RuntimeError(f"seed {seed} already exists")
        if name in self.states_:
            raise RuntimeError(f"rng state {name} already exists")
        self.seeds_.add(seed)
        orig = _get_state(self.cuda)
        if self.cuda:
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states_[name] = _get_state(self.cuda)
        _set_state(orig, self.cuda)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL_RNG):
        if name not in self.states_:
            raise RuntimeError(f"rng state {name} is not added")
        orig = _get_state(self.cuda)
        _set_state(self.states_[name], self.cuda)
        try:
            yield
        finally:
            self.states_[name] = _get_state(self.cuda)
            _set_state(orig, self.cuda)


_TRACKER = RNGStatesTracker()


CudaRNGStatesTracker = RNGStatesTracker          # the reference's name (tensor_parallel/random.py:126)


def get_cuda_rng_tracker() -> RNGStatesTracker:
    return _TRACKER


def get_expert_parallel_rng_tracker_name(): return _EXPERT_PARALLEL_RNG
def get_data_parallel_rng_tracker_name(): return _DATA_PARALLEL_RNG
def get_model_parallel_rng_tracker_name(): return _MODEL_PARALLEL_RNG


def model_parallel_cuda_manual_seed(seed: int, tp_rank: Optional[int] = None, ep_rank: Optional[int] = None,
                                    etp_rank: Optional[int] = None) -> None:
    """Seed the default stream with ``seed`` and register the TP and expert streams."""
    if tp_rank is None:
        tp_rank = state.get_tensor_model_parallel_rank() if state.model_parallel_is_initialized() else 0
    if ep_rank is None:
        ep_rank = state.get_expert_model_parallel_rank() if state.model_parallel_is_initialized() else 0
    if etp_rank is None:
        etp_rank = state.get_expert_tensor_parallel_rank() if state.model_parallel_is_initialized() else 0
    _TRACKER.reset()
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)
    _TRACKER.add(_DATA_PARALLEL_RNG, seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG, seed + 2718 + tp_rank)
    _TRACKER.add(_EXPERT_PARALLEL_RNG, seed + 1024 + 100 * ep_rank + etp_rank)


# ------------------------------------------------------------------ activation checkpointing
class _CheckpointFn(torch.autograd.Function):
    """Recompute ``fn(*args)`` in backward with the RNG streams of the forward pass
    (reference: random.py:407-476)."""

    @staticmethod
    def forward(ctx, fn, n_tensors, *args):
        ctx.fn = fn
        ctx.cuda = torch.cuda.is_available()
        ctx.rng = _get_state(ctx.cuda)
        ctx.cpu_rng = torch.get_rng_state()
        ctx.tracker = _TRACKER.get_states()
        with torch.no_grad():
            out = fn(*args)
        ctx.tensor_idx = [i for i, a in enumerate(args) if torch.is_tensor(a)]
        ctx.others = [None if torch.is_tensor(a) else a for a in args]
        ctx.save_for_backward(*[args[i] for i in ctx.tensor_idx])
        return out

    @staticmethod
    def backward(ctx, *grads):
        saved = ctx.saved_tensors
        args = list(ctx.others)
        for i, t in zip(ctx.tensor_idx, saved):
            d = t.detach()
            d.requires_grad_(t.requires_grad)
            args[i] = d
        cur, cur_cpu, cur_tr = _get_state(ctx.cuda), torch.get_rng_state(), _TRACKER.get_states()
        _set_state(ctx.rng, ctx.cuda)
        torch.set_rng_state(ctx.cpu_rng)
        _TRACKER.set_states(ctx.tracker)
        with torch.enable_grad():
            out = ctx.fn(*args)
        _set_state(cur, ctx.cuda)
        torch.set_rng_state(cur_cpu)
        _TRACKER.set_states(cur_tr)
        outs = (out,) if torch.is_tensor(out) else tuple(out)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(a.grad if torch.is_tensor(a) else None for a in args)


def checkpoint(function, distribute_saved_activations: bool, *args):
    """Run ``function`` without storing its intermediate activations."""
    del distribute_saved_activations   # sharded storage of the input is not needed at these sizes
    return _CheckpointFn.apply(function, len(args), *args)


class CheckpointWithoutOutput:
    """Checkpoint whose *output* is also freed once consumed and re-materialised just
    before the consumer's backward (reference: random.py:521-612).  Usage:

        ck = CheckpointWithoutOutput()
        y = ck.checkpoint(fn, x)
        z = consumer(y)
        ck.discard_output_and_register_recompute(z)
    """

    def __init__(self):
        self.fn = None
        self.args = None
        self.out = None
        self.rng = None

    def checkpoint(self, fn, *args):
        self.fn, self.args = fn, args
        self.cuda = torch.cuda.is_available()
        self.rng = (_get_state(self.cuda), torch.get_rng_state(), _TRACKER.get_states())
        self.inputs = [a.detach().requires_grad_(a.requires_grad) if torch.is_tensor(a) else a for a in args]
        with torch.enable_grad():
            self.out = fn(*self.inputs)
        # hand the consumer a tensor whose storage can be dropped independently of the graph
        return _Passthrough.apply(self, self.out, *[a for a in args if torch.is_tensor(a)])

    def discard_output_and_register_recompute(self, hook_tensor):
        if self.out is not None and torch.is_tensor(self.out):
            self.out.untyped_storage().resize_(0)
        if hook_tensor.requires_grad:
            hook_tensor.register_hook(self._recompute)

    def _recompute(self, _):
        if self.out is None or self.out.untyped_storage().size() > 0:
            return
        cur = (_get_state(self.cuda), torch.get_rng_state(), _TRACKER.get_states())
        _set_state(self.rng[0], self.cuda)
        torch.set_rng_state(self.rng[1])
        _TRACKER.set_states(self.rng[2])
        with torch.no_grad():
            fresh = self.fn(*self.inputs)
        _set_state(cur[0], self.cuda)
        torch.set_rng_state(cur[1])
        _TRACKER.set_states(cur[2])
        self.out.untyped_storage().resize_(fresh.untyped_storage().size())
        self.out.copy_(fresh)


class _Passthrough(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ck, out, *inputs):
        ctx.ck = ck
        return out.detach().view_as(out)

    @staticmethod
    def backward(ctx, g):
        ck = ctx.ck
        ck._recompute(None)
        # the recorded graph of ck.out is intact (storage was only resized), so backprop through it
        torch.autograd.backward(ck.out, g)
        grads = [a.grad for a in ck.inputs if torch.is_tensor(a)]
        return (None, None) + tuple(grads)
