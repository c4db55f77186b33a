"""Cross-rank gradient fix-ups run once per step after backward
(reference: megatron/core/distributed/finalize_model_grads.py:78-361):

1. finish every chunk's data-parallel reduction;
2. all-reduce over the TP group the gradients of parameters that are replicated across TP
   but saw only this rank's sequence shard (norm weights/biases, router weights under
   sequence parallelism);
3. all-reduce the tied word-embedding gradient between the first and last pipeline stage,
   and the position-embedding gradient inside its group;
4. update router expert biases (aux-loss-free balancing);
5. with per-token loss, divide by the global token count (broadcast from the last pipeline
   stage, summed over data-parallel ranks).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import state
from ..ops.optim import scale_


def _unwrap(m):
    while hasattr(m, "module"):
        m = m.module
    return m


def _allreduce_sequence_parallel_grads(model_chunks, config):
    if not (state.model_parallel_is_initialized() and state.get_tensor_model_parallel_world_size() > 1):
        return
    if not (config.sequence_parallel or config.qk_layernorm):
        return
    grads = []
    for chunk in model_chunks:
        for p in _unwrap(chunk).parameters():
            if p.requires_grad and getattr(p, "sequence_parallel", False) and getattr(p, "main_grad", None) is not None:
                grads.append(p.main_grad)
    if not grads:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, group=state.get_tensor_model_parallel_group())
    o = 0
    for g in grads:
        g.copy_(flat[o:o + g.numel()].view_as(g))
        o += g.numel()


def _allreduce_word_embedding_grads(model_chunks, config):
    if not state.model_parallel_is_initialized() or state.get_pipeline_model_parallel_world_size() == 1:
        return
    if not state.is_rank_in_embedding_group(ignore_virtual=True):
        return
    chunk = None
    if state.is_pipeline_first_stage(ignore_virtual=True):
        chunk = model_chunks[0]
    elif state.is_pipeline_last_stage(ignore_virtual=True):
        chunk = model_chunks[-1]
    if chunk is None:
        return
    m = _unwrap(chunk)
    if not getattr(m, "share_embeddings_and_output_weights", False):
        return
    w = m.shared_embedding_or_output_weight()
    if w is not None and getattr(w, "main_grad", None) is not None:
        dist.all_reduce(w.main_grad, group=state.get_embedding_group())


def _allreduce_position_embedding_grads(model_chunks, config):
    # position embeddings live on the first stage only in decoder-only models; nothing to sync
    return


def _update_router_expert_bias(model_chunks, config):
    if not config.moe_router_enable_expert_bias:
        return
    from ..models.moe import TopKRouter, get_updated_expert_bias
    routers = [m for c in model_chunks for m in _unwrap(c).modules() if isinstance(m, TopKRouter)]
    if not routers:
        return
    tpe = torch.stack([r.local_tokens_per_expert for r in routers])
    bias = torch.stack([r.expert_bias for r in routers])
    new = get_updated_expert_bias(tpe, bias, config.moe_router_bias_update_rate)
    for r, b in zip(routers, new):
        r.local_tokens_per_expert.zero_()
        r.expert_bias.copy_(b)


def finalize_model_grads(model_chunks: List[torch.nn.Module], num_tokens: Optional[torch.Tensor] = None) -> None:
    config = _unwrap(model_chunks[0]).config
    for chunk in model_chunks:
        if hasattr(chunk, "finish_grad_sync"):
            chunk.finish_grad_sync()
    _allreduce_sequence_parallel_grads(model_chunks, config)
    _allreduce_word_embedding_grads(model_chunks, config)
    _allreduce_position_embedding_grads(model_chunks, config)
    _update_router_expert_bias(model_chunks, config)
    if num_tokens is not None:
        dev = next(_unwrap(model_chunks[0]).parameters()).device
        num_tokens = num_tokens.to(dev)
        if dist.is_initialized() and state.model_parallel_is_initialized():
            if state.get_pipeline_model_parallel_world_size() > 1:
                dist.broadcast(num_tokens, src=state.get_pipeline_model_parallel_last_rank(),
                               group=state.get_pipeline_model_parallel_group())
            if state.get_data_parallel_world_size(with_context_parallel=True) > 1:
                dist.all_reduce(num_tokens, group=state.get_data_parallel_group(with_context_parallel=True))
        n = float(num_tokens.item())
        if n > 0:
            for chunk in model_chunks:
                if hasattr(chunk, "scale_gradients"):
                    chunk.scale_gradients(1.0 / n)
