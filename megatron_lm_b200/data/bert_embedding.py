"""Embed text with a BERT model: one vector per input line.

    python -m megatron_lm_b200.data.bert_embedding --load <bert ckpt> <model flags> --tokenizer-type \\
        BertWordPieceLowerCase --vocab-file vocab.txt --output-bert-embeddings --input texts.txt --output emb.npy \\
        [--bert-embedder-type megatron|huggingface] [--embed-batch-size 128]

``megatron``: this library's ``BertModel`` run with ``return_embeddings`` - the mean of the final hidden states of
the real tokens between [CLS] and [SEP].  ``huggingface``: a ``transformers`` BERT model named by ``--hf-model``
(mean of the last hidden states over the attention mask).  Texts are sorted by length before batching and the rows are
written back in input order.

Reference: tools/bert_embedding/embed.py (``BertEmbedder`` :218 with ``embed_text_dataset`` / ``embed_text``,
``embed_data_loader`` :98 with the mean over real tokens), huggingface.py (``HuggingfaceEmbedder``), dataset.py
(``BertEmbeddingDataset``: [CLS] tokens [SEP], truncated to the sequence length).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch


class BertEmbeddingDataset(torch.utils.data.Dataset):
    """Texts -> {"text": ids, "padding_mask", "types"} of one length: [CLS] tokens [SEP] padded."""

    def __init__(self, texts: Sequence[str], tokenizer, max_seq_length: int):
        self.texts, self.tok, self.n = list(texts), tokenizer, max_seq_length

    def __len__(self):
        return len(self.texts)

    def __getitem__(self, i):
        ids = list(self.tok.tokenize(self.texts[i]))[: self.n - 2]
        ids = [self.tok.cls] + ids + [self.tok.sep]
        real = len(ids)
        ids = ids + [self.tok.pad] * (self.n - real)
        mask = [1] * real + [0] * (self.n - real)
        return {"text": np.asarray(ids, dtype=np.int64), "padding_mask": np.asarray(mask, dtype=np.int64),
                "types": np.zeros(self.n, dtype=np.int64), "length": real}


class BertEmbedder:
    """``model``: a ``BertModel`` built with ``return_embeddings=True`` (``embedder_type="megatron"``) or a Hugging Face
    encoder returning ``last_hidden_state`` (``"huggingface"``, with its own tokenizer passed as ``tokenizer``)."""

    def __init__(self, model, tokenizer, max_seq_length: int, batch_size: int = 128, embedder_type: str = "megatron",
                 device: Optional[str] = None):
        if embedder_type not in ("megatron", "huggingface"):
            raise ValueError(f"unknown embedder type {embedder_type!r}")
        self.model, self.tok, self.n, self.bs, self.kind = model, tokenizer, max_seq_length, batch_size, embedder_type
        self.device = device or (next(model.parameters()).device if hasattr(model, "parameters") else "cpu")

    @torch.no_grad()
    def embed_text_dataset(self, dataset: BertEmbeddingDataset) -> np.ndarray:
        order = sorted(range(len(dataset)), key=lambda i: dataset[i]["length"])
        out: Optional[np.ndarray] = None
        was_training = getattr(self.model, "training", False)
        self.model.eval()
        for lo in range(0, len(order), self.bs):
            idx = order[lo:lo + self.bs]
            items = [dataset[i] for i in idx]
            longest = max(it["length"] for it in items)
            ids = torch.from_numpy(np.stack([it["text"][:longest] for it in items])).to(self.device)
            mask = torch.from_numpy(np.stack([it["padding_mask"][:longest] for it in items])).to(self.device)
            emb = self.model(ids, mask, torch.zeros_like(ids)).float().cpu().numpy()
            if out is None:
                out = np.zeros((len(dataset), emb.shape[1]), dtype=np.float32)
            out[idx] = emb
        if was_training:
            self.model.train()
        return out if out is not None else np.zeros((0, 0), dtype=np.float32)

    def embed_text(self, text: str) -> np.ndarray:
        return self.embed_texts([text])[0]

    @torch.no_grad()
    def embed_texts(self, texts: Sequence[str]) -> np.ndarray:
        if self.kind == "huggingface":
            out = []
            for lo in range(0, len(texts), self.bs):
                enc = self.tok(list(texts[lo:lo + self.bs]), padding=True, truncation=True, max_length=self.n,
                               return_tensors="pt").to(self.device)
                h = self.model(**enc).last_hidden_state
                m = enc["attention_mask"].unsqueeze(-1).to(h.dtype)
                out.append(((h * m).sum(1) / m.sum(1).clamp(min=1)).float().cpu().numpy())
            return np.concatenate(out) if out else np.zeros((0, 0), dtype=np.float32)
        return self.embed_text_dataset(BertEmbeddingDataset(texts, self.tok, self.n))


def add_embedding_args(parser):
    g = parser.add_argument_group(title="bert embedding")
    g.add_argument("--input", required=True, help="text file, one text per line")
    g.add_argument("--output", required=True, help=".npy file of [lines, hidden] float32")
    g.add_argument("--embed-batch-size", type=int, default=128)
    g.add_argument("--hf-model", default=None, help="model name or directory for --bert-embedder-type huggingface")
    return parser


def main(argv=None, tokenizer=None) -> np.ndarray:
    from ..training import arguments as A
    args = A.parse_args(add_embedding_args, argv=argv)
    if args.micro_batch_size is None:
        args.micro_batch_size = 1
    with open(args.input) as f:
        texts = [line.rstrip("\n") for line in f if line.strip()]
    kind = getattr(args, "bert_embedder_type", "megatron")
    if kind == "huggingface":
        import transformers
        if not args.hf_model:
            raise SystemExit("--bert-embedder-type huggingface needs --hf-model")
        tok = transformers.AutoTokenizer.from_pretrained(args.hf_model)
        model = transformers.AutoModel.from_pretrained(args.hf_model).eval()
        emb = BertEmbedder(model, tok, args.seq_length or 256, args.embed_batch_size, "huggingface", "cpu").embed_texts(texts)
    else:
        if not getattr(args, "output_bert_embeddings", False):
            raise SystemExit("give --output-bert-embeddings: the model is built to return embeddings, not logits")
        args = A.validate_args(args)
        if tokenizer is None:
            from .tokenizer import build_tokenizer
            tokenizer = build_tokenizer(args)
        if args.padded_vocab_size is None:
            args.padded_vocab_size = getattr(tokenizer, "vocab_size", None)
        from ..models.bert import BertModel
        cfg = A.core_transformer_config_from_args(args)
        dev = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
        if dev.type == "cpu":
            cfg.use_cpu_initialization = True
        model = BertModel(cfg, 2, args.padded_vocab_size, args.max_position_embeddings, add_binary_head=True,
                          return_embeddings=True, parallel_output=False).to(dev)
        if args.load is not None:
            from ..training import checkpointing
            checkpointing.load_checkpoint([model], None, None, args, strict=False)
        emb = BertEmbedder(model, tokenizer, args.seq_length, args.embed_batch_size).embed_texts(texts)
    np.save(args.output, emb)
    print(f" embedded {len(texts)} texts into {args.output}: {emb.shape}", flush=True)
    return emb


if __name__ == "__main__":
    main()
