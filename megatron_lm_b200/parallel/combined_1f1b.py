"""Forward of microbatch i interleaved with backward of microbatch i-1 at sub-layer granularity, so that the
expert-parallel token exchange of one direction overlaps the dense compute of the other.

Reference: megatron/core/pipeline_parallel/combined_1f1b.py (``combined_1f1b_schedule_for_no_pipelining`` :24,
``combined_forward_backward_step`` :168), pipeline_parallel/utils.py (``ScheduleNode`` :151, stream handling),
models/common/model_chunk_schedule_plan.py (``TransformerLayerSchedulePlan`` :38,
``TransformerModelChunkSchedulePlan`` :255, ``run`` :352) and models/gpt/fine_grained_callables.py.

A model chunk's forward is cut into *nodes* - embedding, then per layer: attention, (MoE) dispatch, experts,
combine, or (dense) MLP, then the head with the loss.  Each node detaches its inputs, runs on the compute or the
communication stream, and keeps its little autograd graph; ``backward`` of a node runs exactly that graph and
hands the input gradients to the node before it.  ``schedule_chunk_1f1b`` walks the forward nodes of one
microbatch and the backward nodes of the previous one alternately, pairing a communication node of one with a
compute node of the other.  On CPU tensors there are no streams and the order is simply sequential - same
numbers, which is what the tests check.
"""
from __future__ import annotations

import contextlib
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from .layers import _DEFERRED_WGRADS, drain_deferred_wgrads

_COMP, _COMM = None, None


def set_streams(comp=None, comm=None) -> None:
    global _COMP, _COMM
    _COMP, _COMM = comp, comm


def get_comp_stream():
    return _COMP


def get_comm_stream():
    return _COMM


class ScheduleNode:
    """One schedulable piece of a forward pass with its own autograd boundary."""

    def __init__(self, forward_func: Callable, name: str = "", comm: bool = False):
        self.fn, self.name, self.comm = forward_func, name, comm
        self.inputs: Tuple = ()
        self.outputs: Tuple = ()
        self.event = None

    def _stream_ctx(self):
        st = _COMM if self.comm else _COMP
        if st is None or not torch.cuda.is_available():
            return contextlib.nullcontext(), None
        return torch.cuda.stream(st), st

    def forward(self, *inputs):
        ctx, st = self._stream_ctx()
        det = []
        for x in inputs:
            if torch.is_tensor(x) and x.is_floating_point():
                d = x.detach()
                d.requires_grad_(x.requires_grad or torch.is_grad_enabled())
                det.append(d)
            else:
                det.append(x)
        self.inputs = tuple(det)
        with ctx:
            if st is not None:
                st.wait_stream(torch.cuda.current_stream())
            out = self.fn(*det)
            if st is not None:
                self.event = torch.cuda.Event()
                self.event.record(st)
        self.outputs = out if isinstance(out, tuple) else (out,)
        if st is not None:
            torch.cuda.current_stream().wait_event(self.event)
        return out

    def backward(self, *output_grads):
        ctx, st = self._stream_ctx()
        outs, grads = [], []
        for o, g in zip(self.outputs, output_grads):
            if torch.is_tensor(o) and o.requires_grad and g is not None:
                outs.append(o)
                grads.append(g)
        with ctx:
            if st is not None:
                st.wait_stream(torch.cuda.current_stream())
            if outs:
                torch.autograd.backward(outs, grads)
            if st is not None:
                ev = torch.cuda.Event()
                ev.record(st)
                torch.cuda.current_stream().wait_event(ev)
        res = tuple(x.grad if (torch.is_tensor(x) and x.requires_grad) else None for x in self.inputs)
        self.inputs, self.outputs = (), ()            # free the node's graph
        return res


class LayerSchedulePlan:
    """Nodes of one transformer layer.  Dense: [attn, mlp].  MoE: [attn, dispatch, experts, combine]."""

    def __init__(self, layer, rotary=None):
        self.layer = layer
        is_moe = getattr(layer, "is_moe", False)

        def attn(h):
            ln = layer.input_layernorm(h)
            out, bias = layer.self_attention(ln, rotary=rotary)
            return layer._bda(out, bias, h)

        self.nodes: List[ScheduleNode] = [ScheduleNode(attn, f"attn{layer.layer_number}")]
        if not is_moe:
            def mlp(h):
                out, bias = layer.mlp(layer.pre_mlp_layernorm(h))
                return layer._bda(out, bias, h)
            self.nodes.append(ScheduleNode(mlp, f"mlp{layer.layer_number}"))
        else:
            moe = layer.mlp
            state = {}

            def dispatch(h):
                ln = layer.pre_mlp_layernorm(h)
                probs, rmap = moe.router(ln)
                tokens, tpe = moe.token_dispatcher.dispatch(ln, probs, rmap)
                state["tpe"], state["rmap"] = tpe, rmap
                return tokens, h, ln, probs

            def experts(tokens, h, ln, probs):
                out, _ = moe.experts(tokens, state["tpe"])
                return out, h, ln, probs

            def combine(out, h, ln, probs):
                # the router probabilities enter this node as its own input, so that the weighting's gradient
                # flows back through the node boundary instead of reaching into the dispatch node's graph
                d = moe.token_dispatcher
                if getattr(d, "fused", False):
                    rm = state["rmap"].t().contiguous()
                    d.copy_probs = probs.t().contiguous().masked_select(rm)
                elif hasattr(d, "local_probs"):
                    raise NotImplementedError("the interleaved schedule supports the all-to-all dispatchers only")
                else:
                    d.probs = probs
                y = d.combine(out)
                if moe.shared_experts is not None:
                    y = y + moe.shared_experts(ln)
                return layer._bda(y, None, h)

            self.nodes += [ScheduleNode(dispatch, f"dispatch{layer.layer_number}", comm=True),
                           ScheduleNode(experts, f"experts{layer.layer_number}"),
                           ScheduleNode(combine, f"combine{layer.layer_number}", comm=True)]


class ModelChunkSchedulePlan:
    """All nodes of one microbatch through one GPT model chunk, ending in the (scaled) loss."""

    def __init__(self, model, input_ids, position_ids=None, labels=None, loss_func: Optional[Callable] = None):
        m = model
        while hasattr(m, "module") and not hasattr(m, "decoder"):
            m = m.module
        self.model = m
        rotary = None
        if getattr(m, "rotary_pos_emb", None) is not None:
            rotary = m.rotary_pos_emb(input_ids.shape[1], input_ids.device)

        def pre():
            return m.embedding(input_ids, position_ids)

        def post(h):
            if m.decoder.final_layernorm is not None:
                h = m.decoder.final_layernorm(h)
            w = m.shared_embedding_or_output_weight() if m.share_embeddings_and_output_weights else None
            logits, _ = m.output_layer(h, weight=w)
            out = m.compute_language_model_loss(labels, logits) if labels is not None else logits.transpose(0, 1)
            return loss_func(out) if loss_func is not None else out

        self.pre = ScheduleNode(pre, "embedding")
        self.layers = [LayerSchedulePlan(l, rotary) for l in m.decoder.layers]
        self.post = ScheduleNode(post, "head")
        self.hidden = None
        self.loss = None

    def nodes(self) -> List[ScheduleNode]:
        return [self.pre] + [n for l in self.layers for n in l.nodes] + [self.post]


def _run_forward_node(node: ScheduleNode, carry):
    out = node.forward(*carry) if carry is not None else node.forward()
    return out if isinstance(out, tuple) else (out,)


def schedule_chunk_1f1b(f_plan: Optional[ModelChunkSchedulePlan], b_plan: Optional[ModelChunkSchedulePlan],
                        b_loss_grad: Optional[torch.Tensor] = None):
    """Run the forward of ``f_plan`` and the backward of ``b_plan`` interleaved node by node.  Returns the forward
    plan's final output (the loss).  ``b_plan`` must have completed its forward."""
    f_nodes = f_plan.nodes() if f_plan is not None else []
    b_nodes = list(reversed(b_plan.nodes())) if b_plan is not None else []
    f_carry = None
    b_carry: Tuple = (b_loss_grad if b_loss_grad is not None else
                      (torch.ones_like(b_plan.loss) if b_plan is not None else None),)
    fi = bi = 0
    while fi < len(f_nodes) or bi < len(b_nodes):
        # a backward node first (its communication can then hide behind the forward node that follows), then forward
        if bi < len(b_nodes):
            b_carry = b_nodes[bi].backward(*b_carry)
            bi += 1
        if fi < len(f_nodes):
            f_carry = _run_forward_node(f_nodes[fi], f_carry)
            fi += 1
        if _DEFERRED_WGRADS:
            # delay_wgrad_compute: the weight gradients of the backward node above run after the forward node that
            # followed it, i.e. under whatever communication that node started
            drain_deferred_wgrads(0)
    if f_plan is not None:
        f_plan.loss = f_carry[0]
        return f_plan.loss
    return None


def combined_1f1b_schedule_for_no_pipelining(*, forward_step_func, data_iterator, model, num_microbatches: int,
                                             seq_length: int = 0, micro_batch_size: int = 0, forward_only: bool = False,
                                             **_):
    """Drop-in for the no-pipelining schedule when ``overlap_moe_expert_parallel_comm`` is on.
    ``forward_step_func(data_iterator, model, return_schedule_plan=True)`` returns (plan, loss_func) where
    ``loss_func(output) -> (loss, report)`` or ``(loss_sum, num_tokens, report)``."""
    from .schedules import get_model_config
    if isinstance(model, (list, tuple)):
        model = model[0]
    if isinstance(data_iterator, (list, tuple)):
        data_iterator = data_iterator[0]
    config = get_model_config(model)
    no_sync = config.no_sync_func or contextlib.nullcontext
    store: List[dict] = []
    total_tokens = torch.zeros((), dtype=torch.int64)

    def make_plan():
        nonlocal total_tokens
        plan, loss_func = forward_step_func(data_iterator, model, return_schedule_plan=True)
        inner = plan.post.fn

        def post_with_loss(h):
            nonlocal total_tokens
            res = loss_func(inner(h))
            if len(res) == 3:
                loss_sum, ntok, report = res
                total_tokens = total_tokens + ntok.to(total_tokens.device)
                loss = loss_sum if config.calculate_per_token_loss else \
                    loss_sum / torch.clamp(ntok, min=1).to(loss_sum.dtype) / num_microbatches
            else:
                loss, report = res
                loss = loss / num_microbatches
            store.append(report)
            if config.grad_scale_func is not None:
                loss = config.grad_scale_func(loss)
            return loss
        plan.post.fn = post_with_loss
        return plan

    prev = None
    with no_sync():
        for i in range(num_microbatches):
            cur = make_plan()
            last = i == num_microbatches - 1
            if forward_only:
                with torch.no_grad():
                    schedule_chunk_1f1b(cur, None)
                continue
            if last:
                break
            schedule_chunk_1f1b(cur, prev)
            prev = cur
    if not forward_only:
        # the last forward still overlaps the previous backward, but its own backward must synchronise gradients
        schedule_chunk_1f1b(cur, prev)
        schedule_chunk_1f1b(None, cur)
        if config.finalize_model_grads_func is not None:
            config.finalize_model_grads_func([model], total_tokens if config.calculate_per_token_loss else None)
    return store
