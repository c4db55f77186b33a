"""Evidence embeddings for open-domain retrieval: the store the indexer fills, exact maximum-inner-product search
over it, and the evidence dataset that is embedded.

Reference: megatron/legacy/data/realm_index.py (``OpenRetreivalDataStore`` :18: embeddings by row id, one shard file
per data-parallel rank, merged by rank 0; ``FaissMIPSIndex`` :119), megatron/legacy/data/orqa_wiki_dataset.py
(``OpenRetrievalEvidenceDataset`` :122: a tab-separated file ``id, text, title`` with a header line, encoded as
``[CLS] title [SEP] text [SEP]``) and megatron/legacy/indexer.py (``IndexBuilder`` :18).

The search is exact rather than an approximate library index: scores are one matrix product per block of evidence
rows on the device that holds the queries, with a running top-k, so twenty million 128-wide half-precision rows
(5 GB) fit a single GPU's memory many times over and every block is a plain GEMM.
"""
from __future__ import annotations

import csv
import os
import random
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch


class BlockEmbeddingStore:
    """Embeddings by row id.  ``add`` collects, ``save_shard`` writes this rank's part beside the final file,
    ``merge_shards_and_save`` (one rank) joins all parts into ``embedding_path`` and removes them."""

    def __init__(self, embedding_path: Optional[str] = None, load_from_path: bool = False, rank: int = 0,
                 dtype: torch.dtype = torch.float16):
        self.embedding_path, self.rank, self.dtype = embedding_path, rank, dtype
        self.embed_data: Dict[int, torch.Tensor] = {}
        if embedding_path is not None:
            stem = os.path.splitext(embedding_path)[0]
            self.temp_dir = stem + "_tmp"
        if load_from_path:
            self.load_from_file()

    def __len__(self):
        return len(self.embed_data)

    def clear(self):
        self.embed_data = {}

    def state(self) -> Dict[str, torch.Tensor]:
        ids = sorted(self.embed_data)
        embeds = torch.stack([self.embed_data[i] for i in ids]) if ids else torch.empty(0, 0, dtype=self.dtype)
        return {"row_ids": torch.tensor(ids, dtype=torch.int64), "embeds": embeds}

    def _take(self, state):
        for i, e in zip(state["row_ids"].tolist(), state["embeds"]):
            if i in self.embed_data:
                raise ValueError(f"row id {i} was embedded twice")
            self.embed_data[i] = e

    def load_from_file(self):
        self._take(torch.load(self.embedding_path, map_location="cpu", weights_only=True))

    def add_block_data(self, row_ids, embeds: torch.Tensor, allow_overwrite: bool = False):
        embeds = embeds.detach().to("cpu", self.dtype)
        for i, e in zip(torch.as_tensor(row_ids).tolist(), embeds):
            if not allow_overwrite and i in self.embed_data:
                raise ValueError(f"row id {i} was embedded twice")
            self.embed_data[int(i)] = e.clone()

    def save_shard(self):
        os.makedirs(self.temp_dir, exist_ok=True)
        torch.save(self.state(), os.path.join(self.temp_dir, f"{self.rank}.pt"))

    def merge_shards_and_save(self):
        seen = set()
        for name in sorted(os.listdir(self.temp_dir)):
            rank = int(os.path.splitext(name)[0])
            seen.add(rank)
            if rank == self.rank and self.embed_data:
                continue                                    # this rank's rows are in memory already
            self._take(torch.load(os.path.join(self.temp_dir, name), map_location="cpu", weights_only=True))
        torch.save(self.state(), self.embedding_path)
        for name in os.listdir(self.temp_dir):
            os.remove(os.path.join(self.temp_dir, name))
        os.rmdir(self.temp_dir)
        return len(seen)


class MIPSIndex:
    """Exact maximum-inner-product search over a matrix of evidence embeddings."""

    def __init__(self, embed_size: int, store: Optional[BlockEmbeddingStore] = None, device=None,
                 block_rows: int = 1 << 20):
        self.embed_size, self.block_rows = embed_size, block_rows
        self.device = torch.device(device) if device is not None else \
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.reset_index()
        if store is not None:
            self.add_embed_data(store)

    def reset_index(self):
        self.row_ids = torch.empty(0, dtype=torch.int64, device=self.device)
        self.embeds = None

    def __len__(self):
        return int(self.row_ids.numel())

    def add_embed_data(self, store: BlockEmbeddingStore):
        st = store.state()
        self.add(st["row_ids"], st["embeds"])

    def add(self, row_ids: torch.Tensor, embeds: torch.Tensor):
        if embeds.shape[-1] != self.embed_size:
            raise ValueError(f"embeddings are {embeds.shape[-1]} wide, the index {self.embed_size}")
        embeds = embeds.to(self.device)
        self.embeds = embeds if self.embeds is None else torch.cat([self.embeds, embeds.to(self.embeds.dtype)])
        self.row_ids = torch.cat([self.row_ids, torch.as_tensor(row_ids, dtype=torch.int64).to(self.device)])

    @torch.no_grad()
    def search_mips_index(self, query_embeds: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """[queries, embed] -> (scores [queries, k], row ids [queries, k]), best first."""
        if self.embeds is None or len(self) == 0:
            raise ValueError("the index is empty")
        k = min(top_k, len(self))
        # half-precision products on a GPU, fp32 on the host
        work = self.embeds.dtype if self.device.type == "cuda" else torch.float32
        q = query_embeds.to(self.device, work)
        best_s = torch.full((q.shape[0], 0), 0.0, device=self.device, dtype=torch.float32)
        best_i = torch.empty((q.shape[0], 0), device=self.device, dtype=torch.int64)
        for lo in range(0, len(self), self.block_rows):
            block = self.embeds[lo:lo + self.block_rows].to(work)
            s = (q @ block.t()).float()
            kk = min(k, s.shape[1])
            top_s, top_j = s.topk(kk, dim=1)
            best_s = torch.cat([best_s, top_s], dim=1)
            best_i = torch.cat([best_i, self.row_ids[lo + top_j]], dim=1)
            if best_s.shape[1] > k:
                best_s, sel = best_s.topk(k, dim=1)
                best_i = best_i.gather(1, sel)
        order = best_s.argsort(dim=1, descending=True)
        return best_s.gather(1, order), best_i.gather(1, order)


class OpenRetrievalEvidenceDataset(torch.utils.data.Dataset):
    """Rows of a tab-separated evidence file (header line, then ``id <tab> text <tab> title``), each encoded as
    ``[CLS] title [SEP] text [SEP]``, cut and padded to ``max_seq_length``."""

    def __init__(self, datapath: str, tokenizer, max_seq_length: int, sample_rate: float = 1.0, seed: int = 1234):
        self.tokenizer, self.max_seq_length = tokenizer, max_seq_length
        self.samples, self.id2text = self.process_samples_from_single_path(datapath)
        if sample_rate < 1:
            k = int(len(self.samples) * sample_rate)
            self.samples = random.Random(seed).sample(self.samples, k)

    @staticmethod
    def process_samples_from_single_path(filename: str):
        rows, id2text = [], {}
        with open(filename, newline="") as f:
            reader = csv.reader(f, delimiter="\t")
            next(reader, None)
            for row in reader:
                doc_id = int(row[0])
                if doc_id in id2text:
                    raise ValueError(f"document id {doc_id} appears twice in {filename}")
                rows.append({"doc_id": doc_id, "text": row[1], "title": row[2]})
                id2text[doc_id] = (row[1], row[2])
        return rows, id2text

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, idx):
        row = self.samples[idx]
        tk = self.tokenizer
        title, text = tk.tokenize(row["title"]), tk.tokenize(row["text"])
        ids = ([tk.cls] + list(title) + [tk.sep] + list(text))[: self.max_seq_length - 1] + [tk.sep]
        n = len(ids)
        tokens = np.full(self.max_seq_length, tk.pad, dtype=np.int64)
        tokens[:n] = ids
        mask = np.zeros(self.max_seq_length, dtype=np.int64)
        mask[:n] = 1
        return {"row_id": np.int64(row["doc_id"]), "context": tokens, "context_pad_mask": mask,
                "context_types": np.zeros(self.max_seq_length, dtype=np.int64)}


class IndexBuilder:
    """One pass over the evidence: every data-parallel rank embeds its rows with the context tower, writes a shard,
    and the first rank merges the shards into ``embedding_path``."""

    def __init__(self, biencoder, dataset, embedding_path: str, batch_size: int = 128, log_interval: int = 1000,
                 dp_rank: int = 0, dp_size: int = 1, group=None, device=None, log=print):
        self.model, self.dataset = biencoder, dataset
        self.batch_size, self.log_interval = batch_size, log_interval
        self.dp_rank, self.dp_size, self.group, self.log = dp_rank, dp_size, group, log
        self.device = device if device is not None else next(biencoder.parameters()).device
        self.store = BlockEmbeddingStore(embedding_path, rank=dp_rank)
        self.iteration = self.total_processed = 0

    def _batches(self) -> Iterable[Sequence[int]]:
        mine = range(self.dp_rank, len(self.dataset), self.dp_size)
        for lo in range(0, len(mine), self.batch_size):
            yield mine[lo:lo + self.batch_size]

    @torch.no_grad()
    def build_and_save_index(self) -> int:
        import torch.distributed as dist
        was_training = self.model.training
        self.model.eval()
        for idxs in self._batches():
            rows = [self.dataset[i] for i in idxs]
            col = lambda k: torch.as_tensor(np.stack([r[k] for r in rows])).to(self.device)
            embeds = self.model._embed(self.model.context_model, col("context"), col("context_pad_mask"),
                                       col("context_types"))
            self.store.add_block_data(np.stack([r["row_id"] for r in rows]), embeds.float())
            self.iteration += 1
            self.total_processed += len(rows) * self.dp_size
            if self.dp_rank == 0 and self.iteration % self.log_interval == 0:
                self.log(f"Batch {self.iteration:10d} | Total {self.total_processed:10d}")
        self.store.save_shard()
        multi = self.dp_size > 1 and dist.is_available() and dist.is_initialized()
        if multi:
            dist.barrier(group=self.group)
        total = 0
        if self.dp_rank == 0:
            self.store.merge_shards_and_save()
            total = len(self.store)
            if total != len(self.dataset):
                raise RuntimeError(f"{total} rows embedded, the evidence has {len(self.dataset)}")
        self.store.clear()
        if multi:
            dist.barrier(group=self.group)
        self.model.train(was_training)
        return total


def retrieval_topk_accuracy(index: MIPSIndex, query_embeds: torch.Tensor, gold_ids: Sequence[Sequence[int]],
                            ks: Sequence[int] = (1, 5, 20, 100)) -> Dict[int, float]:
    """Share of queries with at least one of their gold rows among the first k results."""
    _, found = index.search_mips_index(query_embeds, max(ks))
    found = found.tolist()
    out = {}
    for k in ks:
        hits = sum(1 for row, gold in zip(found, gold_ids) if set(row[:k]) & set(int(g) for g in gold))
        out[k] = hits / max(len(found), 1)
    return out
