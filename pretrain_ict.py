#!/usr/bin/env python
"""Pre-train a BERT biencoder retriever with the inverse cloze task.

Reference: pretrain_ict.py (model provider :30, in-batch softmax loss with embeddings gathered over the data-
parallel group :77-128, top-k accuracies :131, datasets provider :146).  Data: a sentence-split indexed dataset
(``--data-path``) and, optionally, an indexed dataset with one title per document (``--titles-data-path``).
"""
import os
import sys
from functools import partial

import numpy as np
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from megatron_lm_b200.data.ict_dataset import ICTDataset  # noqa: E402
from megatron_lm_b200.data.indexed_dataset import IndexedDataset  # noqa: E402
from megatron_lm_b200.models.bert import BiEncoderModel  # noqa: E402
from megatron_lm_b200.parallel import state  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.batch import broadcast_data  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    if state.get_pipeline_model_parallel_world_size() > 1:
        raise NotImplementedError("the biencoder is trained without pipeline parallelism")
    print_rank_0("building the biencoder ...")
    model = BiEncoderModel(config, args.padded_vocab_size, args.max_position_embeddings,
                           projection_dim=args.biencoder_projection_dim or (args.ict_head_size or 0),
                           shared_query_context_model=args.biencoder_shared_query_context_model)
    from megatron_lm_b200.training import checkpointing
    from megatron_lm_b200.training.pretrain import argparse_namespace_copy
    if getattr(args, "bert_load", None) and args.load is None:
        # --bert-load: both towers start from a pre-trained BERT checkpoint
        from megatron_lm_b200.models.bert import BertModel
        bert = BertModel(config, 2, args.padded_vocab_size, args.max_position_embeddings, add_binary_head=True)
        ft = argparse_namespace_copy(args, finetune=True, no_load_optim=True, no_load_rng=True)
        checkpointing.load_checkpoint([bert], None, None, ft, load_dir=args.bert_load, strict=False)
        n = model.init_from_bert(bert.state_dict())
        print_rank_0(f"biencoder towers initialised from the BERT checkpoint {args.bert_load} ({n} tensors)")
    elif getattr(args, "ict_load", None) and args.load is None:
        # --ict-load: a trained biencoder to continue from (weights only)
        ft = argparse_namespace_copy(args, finetune=True, no_load_optim=True, no_load_rng=True)
        checkpointing.load_checkpoint([model], None, None, ft, load_dir=args.ict_load, strict=False)
        print_rank_0(f"biencoder loaded from {args.ict_load}")
    return model


class _AllGatherWithGrad(torch.autograd.Function):
    """Embeddings of all data-parallel ranks as in-batch negatives; the gradient of a rank's own rows comes back
    summed over the ranks (reference: pretrain_ict.py:47-75)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = torch.distributed.get_world_size(group)
        out = [torch.empty_like(x) for _ in range(world)]
        torch.distributed.all_gather(out, x.contiguous(), group=group)
        return torch.cat(out, dim=0)

    @staticmethod
    def backward(ctx, g):
        world, rank = torch.distributed.get_world_size(ctx.group), torch.distributed.get_rank(ctx.group)
        g = g.contiguous()
        torch.distributed.all_reduce(g, group=ctx.group)
        n = g.shape[0] // world
        return g[rank * n:(rank + 1) * n], None


def get_batch(data_iterator):
    keys = ["query_tokens", "query_pad_mask", "query_types", "context_tokens", "context_pad_mask", "context_types"]
    data = next(data_iterator) if data_iterator is not None else None
    b = broadcast_data(keys, data, torch.int64)
    return tuple(b[k].long() for k in keys)


def loss_func(output_tensor):
    args = get_args()
    q, c = output_tensor
    group = state.get_data_parallel_group()
    world = torch.distributed.get_world_size(group) if torch.distributed.is_initialized() else 1
    rank = torch.distributed.get_rank(group) if world > 1 else 0
    local = q.shape[0]
    if world > 1:
        q_all, c_all = _AllGatherWithGrad.apply(q, group), _AllGatherWithGrad.apply(c, group)
    else:
        q_all, c_all = q, c
    scores = torch.matmul(q_all.float(), c_all.float().t())
    if args.retriever_score_scaling:
        scores = scores / (q.shape[-1] ** 0.5)
    labels = torch.arange(scores.shape[0], device=scores.device)
    loss = F.cross_entropy(scores, labels)
    validate_loss(loss, args)
    stats = {"retrieval loss": loss.detach()}
    ranks_ = (scores.detach() > scores.detach().diag().unsqueeze(1)).sum(dim=1)        # 0 = the right block wins
    for k in (args.retriever_report_topk_accuracies or []):
        stats[f"top{k}_acc"] = (ranks_ < k).float().mean() * 100.0
    del rank, local
    # every rank computes the loss over the gathered batch; the harness averages losses over data-parallel ranks
    return loss, stats


def forward_step(data_iterator, model):
    qt, qm, qy, ct, cm, cy = get_batch(data_iterator)
    return model(qt, qm, qy, ct, cm, cy), loss_func


def train_valid_test_datasets_provider(num_samples):
    args = get_args()
    tok = args.tokenizer
    blocks = IndexedDataset(args.data_path[0])
    titles = IndexedDataset(args.titles_data_path) if args.titles_data_path else None
    ndocs = len(blocks.document_indices) - 1
    from megatron_lm_b200.data.gpt_dataset import parse_and_normalize_split
    fr = np.cumsum([0.0] + parse_and_normalize_split(args.split))
    out = []
    for i, n in enumerate(num_samples):
        lo, hi = int(round(fr[i] * ndocs)), int(round(fr[i + 1] * ndocs))
        out.append(ICTDataset(blocks, titles, n, args.retriever_seq_length if args.retriever_seq_length <= args.seq_length
                              else args.seq_length, tok.cls, tok.sep, tok.pad, args.query_in_block_prob, args.seed,
                              args.use_one_sent_docs, np.arange(lo, hi)) if hi > lo and n else None)
    return tuple(out)


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step,
             args_defaults={"tokenizer_type": "BertWordPieceLowerCase"})
