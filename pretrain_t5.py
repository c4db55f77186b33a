#!/usr/bin/env python
"""Pre-train T5 (span-corruption encoder-decoder).

Reference: pretrain_t5.py (model_provider :67, get_batch :132, forward_step :199, datasets :229).
"""
import os
import sys
from functools import partial

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from megatron_lm_b200.data.indexed_dataset import IndexedDataset  # noqa: E402
from megatron_lm_b200.data.masked_dataset import MaskedWordPieceDatasetConfig, T5MaskedWordPieceDataset  # noqa: E402
from megatron_lm_b200.models.t5 import T5Model  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.batch import broadcast_data  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    print_rank_0("building T5 model ...")
    enc_cfg = None
    enc_n, dec_n = getattr(args, "encoder_num_layers", None), getattr(args, "decoder_num_layers", None)
    if enc_n or dec_n:
        # --encoder-num-layers / --decoder-num-layers: stacks of different depth (one pipeline stage)
        import copy
        from megatron_lm_b200.parallel import state
        if state.get_pipeline_model_parallel_world_size() > 1:
            raise NotImplementedError("separate encoder / decoder depths with pipeline parallelism")
        enc_cfg = copy.copy(config)
        enc_cfg.num_layers = enc_n or config.num_layers
        config = copy.copy(config)
        config.num_layers = dec_n or config.num_layers
    return T5Model(config, encoder_config=enc_cfg, vocab_size=args.padded_vocab_size, max_sequence_length=args.max_position_embeddings,
                   pre_process=pre_process, post_process=post_process, parallel_output=True,
                   share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                   position_embedding_type=args.position_embedding_type, rotary_percent=args.rotary_percent)


def get_batch(data_iterator):
    keys = ["text_enc", "text_dec", "labels", "loss_mask", "enc_mask", "dec_mask"]
    data = next(data_iterator) if data_iterator is not None else None
    b = broadcast_data(keys, data, torch.int64)
    enc_m, dec_m = b["enc_mask"].float(), b["dec_mask"].float()
    enc_mask = enc_m.unsqueeze(1) * enc_m.unsqueeze(2)
    enc_dec_mask = dec_m.unsqueeze(2) * enc_m.unsqueeze(1)
    return (b["text_enc"].long(), b["text_dec"].long(), b["loss_mask"].float(), b["labels"].long(), enc_mask, None,
            enc_dec_mask)


def loss_func(loss_mask, output_tensor):
    lm = output_tensor.float()
    loss = torch.sum(lm.view(-1) * loss_mask.reshape(-1)) / loss_mask.sum().clamp(min=1)
    validate_loss(loss, get_args())
    return loss, {"lm loss": loss.detach()}


def forward_step(data_iterator, model):
    enc, dec, loss_mask, labels, enc_mask, dec_mask, enc_dec_mask = get_batch(data_iterator)
    out = model(enc, dec, enc_mask, dec_mask, enc_dec_mask, lm_labels=labels.clamp(min=0))
    return out, partial(loss_func, loss_mask)


def train_valid_test_datasets_provider(num_samples):
    args = get_args()
    cfg = MaskedWordPieceDatasetConfig(sequence_length=args.encoder_seq_length, sequence_length_encoder=args.encoder_seq_length,
                                       sequence_length_decoder=args.decoder_seq_length, random_seed=args.seed,
                                       masking_probability=args.mask_prob, short_sequence_probability=args.short_seq_prob,
                                       masking_max_ngram=10, tokenizer=args.tokenizer)
    ds = IndexedDataset(args.data_path[0])
    ndocs = len(ds.document_indices) - 1
    from megatron_lm_b200.data.gpt_dataset import parse_and_normalize_split
    fr = np.cumsum([0.0] + parse_and_normalize_split(args.split))
    out = []
    for i, n in enumerate(num_samples):
        lo, hi = int(round(fr[i] * ndocs)), int(round(fr[i + 1] * ndocs))
        out.append(T5MaskedWordPieceDataset(ds, np.arange(lo, hi), n, ("train", "valid", "test")[i], cfg)
                   if hi > lo and n else None)
    return tuple(out)


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step,
             args_defaults={"tokenizer_type": "BertWordPieceLowerCase", "vocab_extra_ids": 100})
