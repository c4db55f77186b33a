#!/usr/bin/env python
"""Pre-train a Retro (retrieval-enhanced) GPT model.

Reference: pretrain_retro.py (model_provider :62, get_batch :105, forward_step :167, dataset provider :204).
The retrieval data come from ``python -m megatron_lm_b200.data.retro_preprocess`` (``--retro-project-dir`` holds
chunk_db.npz and neighbors.npy); without a project directory they are built in memory from ``--data-path`` at
start-up with the bag-of-tokens embedder, which is enough for small corpora and for tests.

    python pretrain_retro.py --data-path <prefix> --retro-chunk-length 64 --seq-length 2048 ...
"""
import dataclasses
import os
import sys
from functools import partial

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from megatron_lm_b200.data import retro_preprocess as R  # noqa: E402
from megatron_lm_b200.data.indexed_dataset import IndexedDataset  # noqa: E402
from megatron_lm_b200.models.retro import RetroConfig, RetroModel  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def add_retro_args(parser):
    g = parser.add_argument_group(title="retro data")
    g.add_argument("--retro-chunk-length", type=int, default=64)
    return parser


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    print_rank_0("building Retro model ...")
    kw = {f.name: getattr(config, f.name) for f in dataclasses.fields(config) if f.init}
    rcfg = RetroConfig(**kw, retro_chunk_length=args.retro_chunk_length, retro_num_neighbors=args.retro_num_neighbors,
                       retro_num_retrieved_chunks=args.retro_num_retrieved_chunks,
                       retro_encoder_num_layers=args.retro_encoder_layers, retro_project_dir=args.retro_project_dir,
                       retro_attention_gate=getattr(args, "retro_attention_gate", 1.0),
                       retro_encoder_hidden_dropout=getattr(args, "retro_encoder_hidden_dropout", 0.1),
                       retro_encoder_attention_dropout=getattr(args, "retro_encoder_attention_dropout", 0.1))
    for name in ("no_sync_func", "grad_sync_func", "param_sync_func", "finalize_model_grads_func", "grad_scale_func"):
        setattr(rcfg, name, getattr(config, name, None))
    return RetroModel(rcfg, args.padded_vocab_size, args.max_position_embeddings, pre_process=pre_process,
                      post_process=post_process, position_embedding_type=args.position_embedding_type,
                      share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights)


class _Samples(torch.utils.data.Dataset):
    """``n`` samples drawn cyclically from a RetroDataset slice, shaped for next-token prediction."""

    def __init__(self, rd, ids, n):
        self.rd, self.ids, self.n = rd, ids, n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        s = self.rd[int(self.ids[i % len(self.ids)])]
        t = s["text"]
        return {"tokens": t[:-1], "labels": t[1:], "loss_mask": torch.ones(t.numel() - 1),
                "neighbor_tokens": s["neighbor_tokens"]}


def train_valid_test_datasets_provider(num_samples):
    args = get_args()
    ds = IndexedDataset(args.data_path[0])
    proj = args.retro_project_dir
    if proj and os.path.isfile(os.path.join(proj, "chunk_db.npz")):
        db = R.ChunkDB.load(os.path.join(proj, "chunk_db.npz"))
        nb = np.load(os.path.join(proj, "neighbors.npy"))
    else:
        print_rank_0("building the Retro chunk database and neighbours in memory ...")
        db = R.build_chunk_db(ds, args.retro_chunk_length)
        g = torch.Generator().manual_seed(args.seed)
        table = torch.randn(args.padded_vocab_size + 1, 64, generator=g)
        emb = R.embed_chunks(ds, db, R.mean_pool_embedder(table))
        nb = R.query_neighbors(emb, emb, args.retro_num_neighbors, db.doc_ids, db.doc_ids)
    # samples hold seq_length + 1 tokens rounded up to whole chunks; the model sees the first seq_length
    L = args.retro_chunk_length
    rd = R.RetroDataset(ds, db, nb, sample_length=(args.seq_length // L + 1) * L, num_neighbors=args.retro_num_neighbors)
    if len(rd) == 0:
        raise SystemExit("the corpus has no document long enough for one sample")
    from megatron_lm_b200.data.gpt_dataset import parse_and_normalize_split
    fr = np.cumsum([0.0] + parse_and_normalize_split(args.split))
    out = []
    for i, n in enumerate(num_samples):
        lo, hi = int(round(fr[i] * len(rd))), int(round(fr[i + 1] * len(rd)))
        out.append(_Samples(rd, np.arange(lo, max(hi, lo + 1)) % len(rd), n) if n else None)
    return tuple(out)


def loss_func(loss_mask, output_tensor):
    losses = output_tensor.float().view(-1)
    mask = loss_mask.reshape(-1).float()
    loss = torch.sum(losses * mask) / mask.sum().clamp(min=1)
    validate_loss(loss, get_args())
    return loss, {"lm loss": loss.detach()}


def forward_step(data_iterator, model):
    args = get_args()
    b = next(data_iterator)
    dev = torch.cuda.current_device() if torch.cuda.is_available() else "cpu"
    S, L = args.seq_length, args.retro_chunk_length
    tok, lab, lm = b["tokens"][:, :S].to(dev), b["labels"][:, :S].to(dev), b["loss_mask"][:, :S].to(dev)
    ctx = b["neighbor_tokens"][:, :S // L].to(dev)                    # [b, chunks, k, retrieved length]
    out = model(tok, context_input_ids=ctx, labels=lab)
    return out, partial(loss_func, lm)


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step, extra_args_provider=add_retro_args,
             args_defaults={"tokenizer_type": "NullTokenizer"})
