"""Inverse-cloze-task samples for retriever pre-training.

A document of the sentence-split indexed dataset is cut into blocks of consecutive sentences that fit the sequence
length; a sample picks one sentence of a block as the query and the rest of the block (with probability
``query_in_block_prob`` the whole block) as the context, prefixed by the document's title when a titles dataset is
given.  Reference: megatron/legacy/data/ict_dataset.py:44 (``ICTDataset``) with the block mapping the reference
builds in C++ (``helpers.build_blocks_mapping``); here the mapping is a numpy pass over the sentence lengths.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch


def build_blocks_mapping(doc_idx: np.ndarray, sizes: np.ndarray, title_sizes: Optional[np.ndarray], max_seq_length: int,
                         use_one_sent_docs: bool = False) -> np.ndarray:
    """Rows (first sentence, one past last sentence, document, block id): consecutive sentences of a document whose
    token count (plus title and the three special tokens) stays within ``max_seq_length``."""
    rows: List[tuple] = []
    for d in range(len(doc_idx) - 1):
        lo, hi = int(doc_idx[d]), int(doc_idx[d + 1])
        n_sent = hi - lo
        if n_sent < 1 or (n_sent < 2 and not use_one_sent_docs):
            continue
        budget = max_seq_length - 3 - (int(title_sizes[d]) if title_sizes is not None else 0)
        start, used = lo, 0
        for s in range(lo, hi):
            ln = int(sizes[s])
            if used and used + ln > budget:
                if s - start >= (1 if use_one_sent_docs else 2):
                    rows.append((start, s, d, len(rows)))
                start, used = s, 0
            used += ln
        if hi - start >= (1 if use_one_sent_docs else 2):
            rows.append((start, hi, d, len(rows)))
    return np.asarray(rows, dtype=np.int64).reshape(-1, 4)


class ICTDataset(torch.utils.data.Dataset):
    def __init__(self, block_dataset, title_dataset, num_samples: int, max_seq_length: int, cls_id: int, sep_id: int,
                 pad_id: int, query_in_block_prob: float = 0.1, seed: int = 1234, use_one_sent_docs: bool = False,
                 documents: Optional[np.ndarray] = None):
        self.blocks, self.titles = block_dataset, title_dataset
        self.max_seq_length, self.cls, self.sep, self.pad = max_seq_length, cls_id, sep_id, pad_id
        self.query_in_block_prob, self.seed = query_in_block_prob, seed
        doc_idx = np.asarray(block_dataset.document_indices)
        if documents is not None:                                    # a contiguous split of the documents
            lo, hi = int(documents[0]), int(documents[-1]) + 1
            self.doc_base = lo
            doc_idx = doc_idx[lo:hi + 1]
        else:
            self.doc_base = 0
        sizes = np.asarray(block_dataset.sequence_lengths)
        tsz = None
        if title_dataset is not None:
            tsz = np.asarray(title_dataset.sequence_lengths)[self.doc_base:self.doc_base + len(doc_idx) - 1]
        self.mapping = build_blocks_mapping(doc_idx, sizes, tsz, max_seq_length, use_one_sent_docs)
        if len(self.mapping) == 0:
            raise ValueError("no document yields a block (need documents of at least two sentences)")
        self.num_samples = num_samples if num_samples else len(self.mapping)

    def __len__(self):
        return self.num_samples

    def _pad(self, tokens: List[int], title: Optional[List[int]] = None):
        body = ([self.cls] + title + [self.sep] if title else [self.cls]) + tokens
        body = body[: self.max_seq_length - 1] + [self.sep]
        n = len(body)
        ids = np.full(self.max_seq_length, self.pad, dtype=np.int64)
        ids[:n] = body
        mask = np.zeros(self.max_seq_length, dtype=np.int64)
        mask[:n] = 1
        return ids, mask

    def __getitem__(self, idx: int) -> Dict[str, np.ndarray]:
        start, end, doc, block = (int(v) for v in self.mapping[idx % len(self.mapping)])
        rng = np.random.RandomState((self.seed + idx) % (2 ** 32))
        sents = [list(map(int, self.blocks[i])) for i in range(start, end)]
        title = list(map(int, self.titles[self.doc_base + doc])) if self.titles is not None else None
        pick = int(rng.randint(0, len(sents)))
        query = sents[pick]
        if len(sents) > 1 and rng.random_sample() >= self.query_in_block_prob:
            sents = sents[:pick] + sents[pick + 1:]                   # the usual case: the query leaves its block
        context = [t for s in sents for t in s]
        q_ids, q_mask = self._pad(query)
        c_ids, c_mask = self._pad(context, title)
        zeros = np.zeros(self.max_seq_length, dtype=np.int64)
        return {"query_tokens": q_ids, "query_pad_mask": q_mask, "query_types": zeros, "context_tokens": c_ids,
                "context_pad_mask": c_mask, "context_types": zeros, "block_data": np.asarray([start, end, doc, block])}
