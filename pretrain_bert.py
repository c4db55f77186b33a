#!/usr/bin/env python
"""Pre-train BERT (masked LM + optional sentence-order head).

Reference: pretrain_bert.py (model_provider :31, get_batch :73, loss_func :106, forward_step :140,
datasets provider :161).  Data: sentence-split indexed datasets (``preprocess_data --split-sentences``).
"""
import os
import sys
from functools import partial

import numpy as np
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from megatron_lm_b200.data.indexed_dataset import IndexedDataset  # noqa: E402
from megatron_lm_b200.data.masked_dataset import BERTMaskedWordPieceDataset, MaskedWordPieceDatasetConfig  # noqa: E402
from megatron_lm_b200.models.bert import BertModel  # noqa: E402
from megatron_lm_b200.parallel import state  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.batch import broadcast_data  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    print_rank_0("building BERT model ...")
    return BertModel(config, num_tokentypes=2 if args.bert_binary_head else 0, vocab_size=args.padded_vocab_size,
                     max_sequence_length=args.max_position_embeddings, pre_process=pre_process,
                     post_process=post_process, add_binary_head=args.bert_binary_head, parallel_output=True,
                     share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights)


def get_batch(data_iterator):
    keys = ["text", "types", "labels", "is_random", "loss_mask", "padding_mask"]
    data = next(data_iterator) if data_iterator is not None else None
    b = broadcast_data(keys, data, torch.int64)
    return (b["text"].long(), b["types"].long(), b["is_random"].long(), b["loss_mask"].float(), b["labels"].long(),
            b["padding_mask"].long())


def loss_func(loss_mask, sentence_order, output_tensor):
    lm_loss_, sop_logits = output_tensor
    lm_loss = torch.sum(lm_loss_.float().view(-1) * loss_mask.reshape(-1)) / loss_mask.sum().clamp(min=1)
    validate_loss(lm_loss, get_args())
    if sop_logits is not None:
        sop_loss = F.cross_entropy(sop_logits.view(-1, 2).float(), sentence_order.view(-1), ignore_index=-1)
        return lm_loss + sop_loss, {"lm loss": lm_loss.detach(), "sop loss": sop_loss.detach()}
    return lm_loss, {"lm loss": lm_loss.detach()}


def forward_step(data_iterator, model):
    args = get_args()
    tokens, types, sentence_order, loss_mask, lm_labels, padding_mask = get_batch(data_iterator)
    if not args.bert_binary_head:
        types = None
    out = model(tokens, padding_mask, tokentype_ids=types, lm_labels=lm_labels.clamp(min=0))
    return out, partial(loss_func, loss_mask, sentence_order)


def train_valid_test_datasets_provider(num_samples):
    args = get_args()
    cfg = MaskedWordPieceDatasetConfig(sequence_length=args.seq_length, random_seed=args.seed,
                                       masking_probability=args.mask_prob,
                                       short_sequence_probability=args.short_seq_prob,
                                       classification_head=args.bert_binary_head, tokenizer=args.tokenizer)
    ds = IndexedDataset(args.data_path[0])
    ndocs = len(ds.document_indices) - 1
    from megatron_lm_b200.data.gpt_dataset import parse_and_normalize_split
    fr = np.cumsum([0.0] + parse_and_normalize_split(args.split))
    out = []
    for i, n in enumerate(num_samples):
        lo, hi = int(round(fr[i] * ndocs)), int(round(fr[i + 1] * ndocs))
        out.append(BERTMaskedWordPieceDataset(ds, np.arange(lo, hi), n, ("train", "valid", "test")[i], cfg)
                   if hi > lo and n else None)
    return tuple(out)


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step,
             args_defaults={"tokenizer_type": "BertWordPieceLowerCase"})
