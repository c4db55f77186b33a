"""Retro preprocessing: chunk database, chunk embeddings, nearest-neighbour search and the dataset that serves a
training sample together with its retrieved neighbours.

The reference spreads this over tools/retro/preprocess_data.py and megatron/core/datasets/retro/ (``db`` builds the
chunk database :build_db, ``index`` trains / fills a Faiss index, ``query`` looks up the neighbours of every
training chunk, ``RetroDataset`` query/retro_dataset.py:30 joins them).  The stages here are the same, the search is
exact: inner products against the whole database as one GEMM per block of queries (a few million chunks fit a
B200's memory as bf16 embeddings), so no approximate index has to be trained.

* ``build_chunk_db(indexed_dataset, chunk_length)`` -> ``ChunkDB`` (document id, token offset, length per chunk)
* ``embed_chunks(db, embed_fn, batch)`` -> [num_chunks, d] unit-norm embeddings; ``embed_fn(tokens [b, c])`` is any
  encoder, ``mean_pool_embedder(embedding_table)`` the bag-of-tokens one used when no BERT checkpoint is at hand
* ``query_neighbors(queries, database, k, exclude)`` -> [nq, k] chunk ids, never from the query's own document
* ``RetroDataset`` -> ``{"text", "neighbor_tokens" [chunks_per_sample, k, retrieved_length]}``, where a neighbour
  is the found chunk plus its continuation (the next chunk of the same document), as in the paper
* ``python -m megatron_lm_b200.data.retro_preprocess --input <prefix> --output <dir>`` runs the stages to disk
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np
import torch


@dataclass
class ChunkDB:
    doc_ids: np.ndarray        # [n] document of each chunk
    offsets: np.ndarray        # [n] first token of the chunk inside its document
    lengths: np.ndarray        # [n] tokens in the chunk (the last chunk of a document may be short)
    chunk_length: int

    def __len__(self):
        return len(self.doc_ids)

    def save(self, path: str) -> None:
        np.savez(path, doc_ids=self.doc_ids, offsets=self.offsets, lengths=self.lengths,
                 chunk_length=np.int64(self.chunk_length))

    @classmethod
    def load(cls, path: str) -> "ChunkDB":
        z = np.load(path)
        return cls(z["doc_ids"], z["offsets"], z["lengths"], int(z["chunk_length"]))


def _document(ds, d: int) -> np.ndarray:
    """All tokens of document ``d`` (its sequences concatenated)."""
    lo, hi = int(ds.document_indices[d]), int(ds.document_indices[d + 1])
    parts = [np.asarray(ds[i]) for i in range(lo, hi)]
    return np.concatenate(parts) if parts else np.zeros(0, dtype=np.int64)


def build_chunk_db(ds, chunk_length: int = 64, min_chunk_length: int = 1) -> ChunkDB:
    docs, offs, lens = [], [], []
    ndocs = len(ds.document_indices) - 1
    for d in range(ndocs):
        lo, hi = int(ds.document_indices[d]), int(ds.document_indices[d + 1])
        n = int(sum(int(ds.sequence_lengths[i]) for i in range(lo, hi)))
        for o in range(0, n, chunk_length):
            ln = min(chunk_length, n - o)
            if ln >= min_chunk_length:
                docs.append(d)
                offs.append(o)
                lens.append(ln)
    return ChunkDB(np.asarray(docs, dtype=np.int64), np.asarray(offs, dtype=np.int64), np.asarray(lens, dtype=np.int64),
                   chunk_length)


def chunk_tokens(ds, db: ChunkDB, ids, pad: int = 0, length: Optional[int] = None) -> np.ndarray:
    """[len(ids), length] token matrix of the given chunks, right-padded."""
    length = length or db.chunk_length
    out = np.full((len(ids), length), pad, dtype=np.int64)
    cache = {}
    for r, c in enumerate(ids):
        d = int(db.doc_ids[c])
        if d not in cache:
            cache[d] = _document(ds, d)
        o, ln = int(db.offsets[c]), int(db.lengths[c])
        out[r, :min(ln, length)] = cache[d][o:o + min(ln, length)]
    return out


# ----------------------------------------------------------------------------- embeddings and search
def mean_pool_embedder(table: torch.Tensor, pad: int = 0) -> Callable[[torch.Tensor], torch.Tensor]:
    """tokens [b, c] -> mean of the rows of ``table`` over the non-pad tokens (a bag-of-tokens encoder)."""
    def fn(tokens: torch.Tensor) -> torch.Tensor:
        m = (tokens != pad).unsqueeze(-1).to(table.dtype)
        e = table[tokens.clamp(min=0, max=table.shape[0] - 1)] * m
        return e.sum(1) / m.sum(1).clamp(min=1)
    return fn


def bert_embedder(model, pad: int = 0) -> Callable[[torch.Tensor], torch.Tensor]:
    """Mean-pooled final hidden states of a BERT-style encoder taking (tokens, padding mask)."""
    def fn(tokens: torch.Tensor) -> torch.Tensor:
        mask = (tokens != pad).long()
        with torch.no_grad():
            h = model(tokens, mask)
        h = h[0] if isinstance(h, tuple) else h
        if h.shape[0] != tokens.shape[0]:
            h = h.transpose(0, 1)
        m = mask.unsqueeze(-1).to(h.dtype)
        return (h * m).sum(1) / m.sum(1).clamp(min=1)
    return fn


def embed_chunks(ds, db: ChunkDB, embed_fn: Callable, batch: int = 1024, device: str = "cpu", pad: int = 0,
                 dtype=torch.float32) -> torch.Tensor:
    out = []
    for s in range(0, len(db), batch):
        ids = range(s, min(s + batch, len(db)))
        t = torch.from_numpy(chunk_tokens(ds, db, ids, pad)).to(device)
        e = embed_fn(t).float()
        out.append(torch.nn.functional.normalize(e, dim=-1).to(dtype))
    return torch.cat(out) if out else torch.zeros(0, 0)


def query_neighbors(queries: torch.Tensor, database: torch.Tensor, k: int, query_docs: np.ndarray,
                    database_docs: np.ndarray, block: int = 4096) -> np.ndarray:
    """Exact top-k by inner product, one GEMM per block of queries; chunks of the query's own document are
    excluded (a sample must not retrieve its own continuation).  Returns [nq, k] database chunk ids (-1 when
    fewer than k candidates exist)."""
    nq = queries.shape[0]
    out = np.full((nq, k), -1, dtype=np.int64)
    ddocs = torch.as_tensor(database_docs, device=database.device)
    for s in range(0, nq, block):
        q = queries[s:s + block].to(database.device, database.dtype)
        sim = (q @ database.t()).float()
        own = torch.as_tensor(query_docs[s:s + block], device=database.device).unsqueeze(1) == ddocs.unsqueeze(0)
        sim = sim.masked_fill(own, float("-inf"))
        kk = min(k, database.shape[0])
        val, idx = torch.topk(sim, kk, dim=1)
        idx = idx.masked_fill(~torch.isfinite(val), -1)
        out[s:s + q.shape[0], :kk] = idx.cpu().numpy()
    return out


# ----------------------------------------------------------------------------- dataset
class RetroDataset(torch.utils.data.Dataset):
    """GPT samples of ``sample_length`` tokens, each with the neighbours of its chunks.

    ``neighbors`` [num_chunks, k] comes from ``query_neighbors`` over the same chunk database; the retrieved text of
    a neighbour is that chunk followed by the next chunk of the same document (2 x chunk_length tokens)."""

    def __init__(self, ds, db: ChunkDB, neighbors: np.ndarray, sample_length: int, num_neighbors: int = 2, pad: int = 0):
        if sample_length % db.chunk_length:
            raise ValueError("sample length must be a multiple of the chunk length")
        self.ds, self.db, self.nb, self.pad = ds, db, neighbors, pad
        self.k = num_neighbors
        self.cps = sample_length // db.chunk_length
        self.sample_length = sample_length
        # samples are runs of ``cps`` consecutive full chunks inside one document
        starts = []
        n = len(db)
        i = 0
        while i + self.cps <= n:
            same = db.doc_ids[i] == db.doc_ids[i + self.cps - 1]
            full = (db.lengths[i:i + self.cps] == db.chunk_length).all()
            cont = db.offsets[i + self.cps - 1] - db.offsets[i] == (self.cps - 1) * db.chunk_length
            if same and full and cont:
                starts.append(i)
                i += self.cps
            else:
                i += 1
        self.starts = np.asarray(starts, dtype=np.int64)

    def __len__(self):
        return len(self.starts)

    def _retrieved(self, c: int) -> np.ndarray:
        L = self.db.chunk_length
        out = np.full(2 * L, self.pad, dtype=np.int64)
        if c < 0:
            return out
        out[:L] = chunk_tokens(self.ds, self.db, [c], self.pad)[0]
        if c + 1 < len(self.db) and self.db.doc_ids[c + 1] == self.db.doc_ids[c]:
            out[L:] = chunk_tokens(self.ds, self.db, [c + 1], self.pad)[0]
        return out

    def __getitem__(self, i):
        c0 = int(self.starts[i])
        text = chunk_tokens(self.ds, self.db, range(c0, c0 + self.cps), self.pad).reshape(-1)
        nbr = np.stack([np.stack([self._retrieved(int(c)) for c in self.nb[c0 + j, :self.k]]) for j in range(self.cps)])
        return {"text": torch.from_numpy(text), "neighbor_tokens": torch.from_numpy(nbr),
                "neighbor_chunks": torch.from_numpy(self.nb[c0:c0 + self.cps, :self.k].copy())}


# ----------------------------------------------------------------------------- command line
def main(argv=None):
    from .indexed_dataset import IndexedDataset
    ap = argparse.ArgumentParser(description="Build the Retro chunk database, embeddings and neighbour table.")
    ap.add_argument("--input", required=True, help="prefix of an indexed dataset (.bin/.idx)")
    ap.add_argument("--output", required=True, help="directory for chunk_db.npz, embeddings.pt, neighbors.npy")
    ap.add_argument("--chunk-length", type=int, default=64)
    ap.add_argument("--num-neighbors", type=int, default=2)
    ap.add_argument("--vocab-size", type=int, required=True)
    ap.add_argument("--embed-dim", type=int, default=256)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    os.makedirs(a.output, exist_ok=True)
    ds = IndexedDataset(a.input)
    db = build_chunk_db(ds, a.chunk_length)
    db.save(os.path.join(a.output, "chunk_db.npz"))
    g = torch.Generator().manual_seed(a.seed)
    table = torch.randn(a.vocab_size + 1, a.embed_dim, generator=g).to(a.device)     # random projection of token counts
    emb = embed_chunks(ds, db, mean_pool_embedder(table), device=a.device,
                       dtype=torch.bfloat16 if a.device != "cpu" else torch.float32)
    torch.save(emb.cpu(), os.path.join(a.output, "embeddings.pt"))
    nb = query_neighbors(emb, emb, a.num_neighbors, db.doc_ids, db.doc_ids)
    np.save(os.path.join(a.output, "neighbors.npy"), nb)
    with open(os.path.join(a.output, "retro.json"), "w") as f:
        json.dump({"chunks": len(db), "chunk_length": a.chunk_length, "num_neighbors": a.num_neighbors,
                   "embed_dim": a.embed_dim}, f)
    print(f"{len(db)} chunks, {a.num_neighbors} neighbours each -> {a.output}")


if __name__ == "__main__":
    main()
