"""Forward/backward schedules: no pipelining, 1F1B, and interleaved 1F1B.

Contracts kept from the reference (megatron/core/pipeline_parallel/schedules.py):
``get_forward_backward_func`` (:31-123) picks the schedule from the pipeline sizes;
``forward_step_func(data_iterator, model)`` returns ``(output, loss_func)`` and
``loss_func(output)`` returns ``(loss, report)`` or ``(loss_sum, num_tokens, report)``
(:185-256); only the last microbatch of a model chunk syncs gradients (:454-579);
warm-up counts and the virtual-microbatch order of the interleaved schedule are
those of :623-730.

The executor is table driven: the whole per-rank sequence of (forward | backward,
chunk, microbatch) steps, with the p2p transfers each step needs, is generated
up front by ``build_pipeline_plan`` and then replayed; the plan is pure Python
data, so the ordering rules are unit-tested without any communication.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Callable, Iterator, List, Optional, Sequence, Tuple, Union

import torch

from . import p2p, state


# ----------------------------------------------------------------------------- plan
_WARM_PIPELINE_GROUPS = set()


def get_pp_rank_microbatches(num_microbatches: int, num_model_chunks: int, microbatch_group_size: int,
                             pp_size: int, pp_rank: int, forward_only: bool = False):
    """(total virtual microbatches, all_warmup, warm-up count, remaining)
    (reference: schedules.py:623-672)."""
    total = num_microbatches * num_model_chunks
    all_warmup = False
    if forward_only:
        warmup = total
    elif num_model_chunks > 1:
        warmup = (pp_size - pp_rank - 1) * 2 + (num_model_chunks - 1) * microbatch_group_size
    else:
        warmup = pp_size - pp_rank - 1
    if warmup >= total:
        warmup, all_warmup = total, True
    return total, all_warmup, warmup, total - warmup


def get_schedule_table(num_microbatches: int, num_model_chunks: int, microbatch_group_size: int):
    """virtual microbatch id -> (microbatch id, chunk id): microbatches are taken in groups of
    ``microbatch_group_size``; inside a group every microbatch goes through chunk 0, then every
    one through chunk 1, and so on (reference: schedules.py:675-702)."""
    table = []
    for lo in range(0, num_microbatches, microbatch_group_size):
        hi = min(lo + microbatch_group_size, num_microbatches)
        for chunk in range(num_model_chunks):
            table += [(mb, chunk) for mb in range(lo, hi)]
    return table


def convert_schedule_table_to_order(num_warmup: int, num_model_chunks: int, schedule_table):
    """1-based signed chunk ids in execution order: +c forward of chunk c-1, -c backward of
    the mirrored chunk (reference: schedules.py:705-730)."""
    _, chunk_ids = zip(*schedule_table)
    fwd = [c + 1 for c in chunk_ids]
    bwd = [c - num_model_chunks for c in chunk_ids]
    order = fwd[:num_warmup]
    for i in range(num_warmup, len(fwd)):
        order.append(fwd[i])
        order.append(bwd[i - num_warmup])
    order.extend(bwd[len(fwd) - num_warmup:] if num_warmup > 0 else [])
    return order


@dataclass
class Step:
    kind: str            # "F" or "B"
    chunk: int
    microbatch: int
    virtual_id: int


def build_pipeline_plan(num_microbatches: int, pp_size: int, pp_rank: int, num_model_chunks: int = 1,
                        microbatch_group_size: Optional[int] = None, forward_only: bool = False) -> List[Step]:
    """The ordered compute steps of one rank for one iteration."""
    g = microbatch_group_size or pp_size
    total, _all, warmup, remaining = get_pp_rank_microbatches(num_microbatches, num_model_chunks, g, pp_size, pp_rank,
                                                              forward_only)
    table = get_schedule_table(num_microbatches, num_model_chunks, g) if num_model_chunks > 1 else \
        [(mb, 0) for mb in range(num_microbatches)]

    def fstep(k):
        mb, c = table[k]
        return Step("F", c, mb, k)

    def bstep(k):
        mb, c = table[k]
        return Step("B", num_model_chunks - 1 - c, mb, k)

    plan = [fstep(k) for k in range(warmup)]
    if forward_only:
        return plan
    for k in range(remaining):
        plan.append(fstep(warmup + k))
        plan.append(bstep(k))
    plan += [bstep(k) for k in range(remaining, total)]
    return plan


# ----------------------------------------------------------------------------- step helpers
def deallocate_output_tensor(out, deallocate: bool = False):
    """Drop an activation's data once it has been sent downstream: only its ``grad_fn`` is needed for this stage's
    backward.  ``.data`` is swapped for a one-element tensor (the send keeps its own reference to the storage until
    it completes); backward then goes through :func:`custom_backward`, which does not compare shapes
    (reference: pipeline_parallel/schedules.py:126-143)."""
    if out is None or not deallocate:
        return
    assert isinstance(out, torch.Tensor) and out._base is None, "only a stage output that is no view can be dropped"
    out.data = torch.empty((1,), device=out.device, dtype=out.dtype)


def custom_backward(output: torch.Tensor, grad_output: Optional[torch.Tensor]) -> None:
    """Run the autograd engine from ``output`` with ``grad_output`` without the shape check of
    ``torch.autograd.backward`` - the output's data has been dropped by :func:`deallocate_output_tensor`
    (reference: pipeline_parallel/schedules.py:146-176)."""
    assert output.numel() == 1, "custom_backward is for outputs whose data was dropped"
    if grad_output is None:
        grad_output = torch.ones_like(output, memory_format=torch.preserve_format)
    from torch.autograd import Variable
    Variable._execution_engine.run_backward(tensors=(output,), grad_tensors=(grad_output,), keep_graph=False,
                                            create_graph=False, inputs=tuple(), allow_unreachable=True,
                                            accumulate_grad=True)


def forward_step(forward_step_func, data_iterator, model, num_microbatches, input_tensor, forward_data_store,
                 config, collect_non_loss_data=False, is_last_stage=True, current_microbatch=None,
                 is_first_microbatch=False):
    """One microbatch forward.  Returns (output tensor or scaled loss, num_tokens)."""
    if hasattr(model, "set_input_tensor"):
        model.set_input_tensor(input_tensor)
    elif hasattr(model, "module") and hasattr(model.module, "set_input_tensor"):
        model.module.set_input_tensor(input_tensor)
    ctx = torch.autocast("cuda", dtype=config.autocast_dtype) if config.enable_autocast else contextlib.nullcontext()
    with ctx:
        output, loss_func = forward_step_func(data_iterator, model)
    num_tokens = torch.zeros((), dtype=torch.int64)
    # Auxiliary losses (MoE load balance / z-loss, MTP) inject their gradient on whichever pipeline stage holds the
    # layer, so their scale (loss scale, divided by the microbatch count) is set on every stage, not only where
    # the main loss is formed (reference: pipeline_parallel/schedules.py:224-238).
    if getattr(config, "num_moe_experts", None) or getattr(config, "mtp_num_layers", None):
        dev = output.device if torch.is_tensor(output) else None
        one = torch.ones(1, device=dev)
        scale = config.grad_scale_func(one) if config.grad_scale_func is not None else one
        scale = scale if config.calculate_per_token_loss else scale / num_microbatches
        if getattr(config, "num_moe_experts", None):
            from ..models.moe import MoEAuxLossAutoScaler
            MoEAuxLossAutoScaler.set_loss_scale(scale)
        if getattr(config, "mtp_num_layers", None):
            from ..models.mtp import MTPLossAutoScaler
            MTPLossAutoScaler.set_loss_scale(scale)
    if is_last_stage:
        if collect_non_loss_data:
            forward_data_store.append(loss_func(output, non_loss_data=True))
            return output, num_tokens
        res = loss_func(output)
        if len(res) == 3:
            loss_sum, num_tokens, report = res
            if not config.calculate_per_token_loss:
                loss = loss_sum / torch.clamp(num_tokens, min=1).to(loss_sum.dtype) / num_microbatches
            else:
                loss = loss_sum
        else:
            loss, report = res
            loss = loss / num_microbatches
        forward_data_store.append(report)
        if config.grad_scale_func is not None:
            loss = config.grad_scale_func(loss)
        return loss, num_tokens
    return output, num_tokens


def backward_step(input_tensor, output_tensor, output_tensor_grad, config):
    """One microbatch backward.  Returns the gradient w.r.t. the stage input (or None)."""
    if input_tensor is not None and input_tensor.requires_grad:
        input_tensor.retain_grad()
    if output_tensor_grad is None:
        torch.autograd.backward(output_tensor)
    elif config.deallocate_pipeline_outputs and output_tensor.numel() == 1 and output_tensor_grad.numel() != 1:
        custom_backward(output_tensor, output_tensor_grad)
    else:
        torch.autograd.backward(output_tensor, output_tensor_grad)
    g = None
    if input_tensor is not None:
        g = input_tensor.grad
    return g


def _call_chunk_hook(hook, chunk: int) -> None:
    """``hook`` is None, one callable (single chunk) or a list with one callable per model chunk."""
    if hook is None:
        return
    if isinstance(hook, (list, tuple)):
        if chunk < len(hook) and hook[chunk] is not None:
            hook[chunk]()
    elif chunk == 0:
        hook()


def _as_list(x):
    return x if isinstance(x, (list, tuple)) else [x]


# ----------------------------------------------------------------------------- no pipelining
def forward_backward_no_pipelining(*, forward_step_func, data_iterator, model, num_microbatches: int,
                                   seq_length: int = 0, micro_batch_size: int = 0, decoder_seq_length=None,
                                   forward_only: bool = False, collect_non_loss_data: bool = False,
                                   first_val_step=None, adjust_tensor_shapes_fn=None):
    """All microbatches forward+backward on one stage; gradient sync only on the last one
    (reference: schedules.py:454-579)."""
    if isinstance(model, (list, tuple)):
        assert len(model) == 1, "no-pipelining schedule takes one model chunk"
        model = model[0]
    if isinstance(data_iterator, (list, tuple)):
        data_iterator = data_iterator[0]
    config = get_model_config(model)
    no_sync = config.no_sync_func or contextlib.nullcontext
    store = []
    total_tokens = torch.zeros((), dtype=torch.int64)

    def run(i, last):
        nonlocal total_tokens
        out, ntok = forward_step(forward_step_func, data_iterator, model, num_microbatches, None, store, config,
                                 collect_non_loss_data, True, i, i == 0)
        total_tokens = total_tokens + ntok.to(total_tokens.device)
        if not forward_only:
            backward_step(None, out, None, config)

    with no_sync():
        for i in range(num_microbatches - 1):
            run(i, False)
    run(num_microbatches - 1, True)
    if config.finalize_model_grads_func is not None and not forward_only:
        config.finalize_model_grads_func([model], total_tokens if config.calculate_per_token_loss else None)
    return store


def get_model_config(model):
    m = model
    while not hasattr(m, "config") and hasattr(m, "module"):
        m = m.module
    return m.config


# ----------------------------------------------------------------------------- pipelined
def get_tensor_shapes(seq_length: int, micro_batch_size: int, config) -> Tuple[int, int, int]:
    """Shape of the activation exchanged between stages: [s / cp / (tp if SP), mbs, h]
    (reference: schedules.py:1653-1700)."""
    s = seq_length // config.context_parallel_size
    if config.sequence_parallel:
        s //= config.tensor_model_parallel_size
    return (s, micro_batch_size, config.hidden_size)


def forward_backward_pipelining(*, forward_step_func, data_iterator, model, num_microbatches: int, seq_length: int,
                                micro_batch_size: int, decoder_seq_length=None, forward_only: bool = False,
                                collect_non_loss_data: bool = False, first_val_step=None,
                                adjust_tensor_shapes_fn=None):
    """1F1B, plain (one chunk) or interleaved (several chunks), driven by ``build_pipeline_plan``.

    Communication per step (all NCCL point-to-point on the pipeline group):
      before F(chunk c): receive the activation unless this is the first virtual stage
      after  F(chunk c): send the output unless this is the last virtual stage
      before B(chunk c): receive the output gradient unless last virtual stage
      after  B(chunk c): send the input gradient unless first virtual stage
    Receives for the *next* step are posted before the current step's compute when
    ``overlap_p2p_comm`` is set, so transfers hide behind compute."""
    chunks = list(model) if isinstance(model, (list, tuple)) else [model]
    iters = list(data_iterator) if isinstance(data_iterator, (list, tuple)) else [data_iterator] * len(chunks)
    v = len(chunks)
    config = get_model_config(chunks[0])
    pp_size = state.get_pipeline_model_parallel_world_size()
    pp_rank = state.get_pipeline_model_parallel_rank()
    if v > 1 and num_microbatches % config.microbatch_group_size_per_vp_stage != 0 and \
            num_microbatches < config.microbatch_group_size_per_vp_stage:
        raise RuntimeError("interleaved schedule needs at least microbatch_group_size_per_vp_stage microbatches")
    plan = build_pipeline_plan(num_microbatches, pp_size, pp_rank, v, config.microbatch_group_size_per_vp_stage,
                               forward_only)
    shape = get_tensor_shapes(seq_length, micro_batch_size, config)
    # a wrapper that sends more than one activation per boundary (distillation: student and teacher hidden states
    # side by side) widens the exchanged tensor (reference: schedules.py adjust_tensor_shapes_fn)
    adjust = adjust_tensor_shapes_fn or getattr(config, "adjust_tensor_shapes_fn", None)
    if adjust is not None:
        shape = tuple(adjust(shape))
    dtype = config.pipeline_dtype or config.params_dtype
    pp_group = state.get_pipeline_model_parallel_group()
    comm = p2p.P2PCommunicator(pp_group, pp_rank, pp_size, shape, dtype, config)
    if pp_group is not None and id(pp_group) not in _WARM_PIPELINE_GROUPS:
        # build the channel communicators before the first step, then line the ranks up again: the ranks of one
        # stage must enter their first step within the wait limit of the fused tensor-parallel kernels
        _WARM_PIPELINE_GROUPS.add(id(pp_group))
        comm.warmup()
        torch.distributed.barrier()

    def first_virtual(c): return pp_rank == 0 and c == 0
    def last_virtual(c): return pp_rank == pp_size - 1 and c == v - 1

    inputs = [[] for _ in range(v)]      # per chunk FIFO of (input_tensor, output_tensor)
    store = []
    total_tokens = torch.zeros((), dtype=torch.int64)
    no_sync_ctx = None
    fwd_count = [0] * v
    bwd_count = [0] * v

    def enter_no_sync():
        nonlocal no_sync_ctx
        if config.no_sync_func is not None and no_sync_ctx is None:
            fn = config.no_sync_func
            if isinstance(fn, (list, tuple)):
                stack = contextlib.ExitStack()
                for f in fn:
                    stack.enter_context(f())
                no_sync_ctx = stack
            else:
                no_sync_ctx = fn()
                no_sync_ctx.__enter__()

    def exit_no_sync():
        nonlocal no_sync_ctx
        if no_sync_ctx is not None:
            if isinstance(no_sync_ctx, contextlib.ExitStack):
                no_sync_ctx.close()
            else:
                no_sync_ctx.__exit__(None, None, None)
            no_sync_ctx = None

    if not forward_only:
        enter_no_sync()
    # pre-post the receive of the very first step
    pending = {}          # step index -> tensor being received

    def post_recv(idx):
        if idx >= len(plan) or idx in pending:
            return
        st = plan[idx]
        if st.kind == "F":
            pending[idx] = None if first_virtual(st.chunk) else comm.irecv_forward()
        else:
            pending[idx] = None if last_virtual(st.chunk) else comm.irecv_backward()

    post_recv(0)
    for idx, st in enumerate(plan):
        c = st.chunk
        if config.overlap_p2p_comm:
            post_recv(idx + 1)
        recv = pending.pop(idx, None)
        if idx not in pending and recv is None and not (
                (st.kind == "F" and first_virtual(c)) or (st.kind == "B" and last_virtual(c))):
            post_recv(idx)
            recv = pending.pop(idx)
        tensor_in = comm.wait(recv) if recv is not None else None
        if v > 1:
            state.set_virtual_pipeline_model_parallel_rank(c)
        if st.kind == "F":
            if tensor_in is not None:
                tensor_in.requires_grad_(not forward_only)
            is_last = last_virtual(c)
            out, ntok = forward_step(forward_step_func, iters[c], chunks[c], num_microbatches, tensor_in, store,
                                     config, collect_non_loss_data, is_last, st.microbatch, fwd_count[c] == 0)
            fwd_count[c] += 1
            total_tokens = total_tokens + ntok.to(total_tokens.device)
            if fwd_count[c] == 1 and c + 1 < v:
                # first microbatch of this chunk: start gathering the next chunk's updated weights behind it
                _call_chunk_hook(config.param_sync_func, c + 1)
            if not is_last:
                comm.send_forward(out)
            if not forward_only:
                inputs[c].append((tensor_in, out))
                if not is_last:
                    deallocate_output_tensor(out, config.deallocate_pipeline_outputs)
        else:
            tensor_in_f, out = inputs[c].pop(0)
            bwd_count[c] += 1
            # the last backward of a chunk is the one that syncs that chunk's gradients
            if bwd_count[c] == num_microbatches:
                exit_no_sync()
            grad_in = backward_step(tensor_in_f, out, tensor_in, config)
            if config.defer_embedding_wgrad_compute:
                # postponed output-layer weight gradients: all of them once this chunk's last backward pass is done
                # (before its gradients are reduced), otherwise only what exceeds the deferral limit
                from .layers import drain_deferred_wgrads
                done = bwd_count[c] == num_microbatches
                drain_deferred_wgrads(0 if done else (config.wgrad_deferral_limit or num_microbatches))
            if bwd_count[c] == num_microbatches:
                # this chunk's gradients are complete: launch whatever part of its data-parallel reduction the
                # per-bucket triggers have not started yet, so it overlaps the other chunks' remaining backward
                # passes (reference: pipeline_parallel/schedules.py:1106-1116)
                _call_chunk_hook(config.grad_sync_func, c)
                if sum(bwd_count) < num_microbatches * v:
                    enter_no_sync()
            if not first_virtual(c):
                comm.send_backward(grad_in)
    comm.drain()
    exit_no_sync()
    if v > 1:
        state.set_virtual_pipeline_model_parallel_rank(0)
    if config.finalize_model_grads_func is not None and not forward_only:
        config.finalize_model_grads_func(chunks, total_tokens if config.calculate_per_token_loss else None)
    return store


def forward_backward_pipelining_with_interleaving(**kw):
    return forward_backward_pipelining(**kw)


def forward_backward_pipelining_without_interleaving(**kw):
    return forward_backward_pipelining(**kw)


def get_forward_backward_func() -> Callable:
    """Pick the schedule for the current pipeline configuration."""
    pp = state.get_pipeline_model_parallel_world_size() if state.model_parallel_is_initialized() else 1
    if pp > 1:
        if state.get_virtual_pipeline_model_parallel_world_size() is not None:
            return forward_backward_pipelining_with_interleaving
        return forward_backward_pipelining_without_interleaving
    return forward_backward_no_pipelining
