"""Masked-language-model datasets for BERT and T5 over sentence-level indexed data.

Reference: megatron/core/datasets/masked_dataset.py (``MaskedWordPieceDataset`` :81, span masking
:238-420), bert_dataset.py (``BERTMaskedWordPieceDataset`` :39), t5_dataset.py
(``T5MaskedWordPieceDataset`` :52).  Samples are runs of consecutive sentences chosen by the C++
``build_mapping`` helper (start sentence, end sentence, target length); masking picks n-gram spans until
``masking_probability`` of the tokens are covered, replacing 80 % by [MASK], 10 % by a random token
and keeping 10 %.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch

from . import helpers


@dataclass
class MaskedWordPieceDatasetConfig:
    sequence_length: int = 512
    random_seed: int = 1234
    masking_probability: float = 0.15
    short_sequence_probability: float = 0.1
    masking_max_ngram: int = 3
    masking_do_full_word: bool = True
    masking_do_permutation: bool = False
    masking_use_longer_ngrams: bool = False
    masking_use_geometric_distribution: bool = False
    classification_head: bool = True          # BERT: sentence-order prediction pairs
    sequence_length_encoder: Optional[int] = None    # T5
    sequence_length_decoder: Optional[int] = None
    tokenizer: object = None


class MaskedWordPieceDataset(torch.utils.data.Dataset):
    def __init__(self, indexed_dataset, indexed_indices: np.ndarray, num_samples: Optional[int], index_split: str,
                 config: MaskedWordPieceDatasetConfig, min_sentences: int = 1, extra_tokens: int = 2):
        self.dataset, self.indices, self.num_samples, self.config = indexed_dataset, indexed_indices, num_samples, config
        tok = config.tokenizer
        self.cls, self.sep, self.mask, self.pad = tok.cls, tok.sep, tok.mask, tok.pad
        self.vocab_size = tok.vocab_size
        docs = np.asarray(indexed_dataset.document_indices, dtype=np.int64)
        lo, hi = int(indexed_indices[0]), int(indexed_indices[-1]) + 1
        docs = np.concatenate((docs[lo:hi], docs[hi:hi + 1])) if hi < len(docs) else docs[lo:]
        sizes = np.asarray(indexed_dataset.sequence_lengths, dtype=np.int32)
        n = num_samples if num_samples is not None else np.iinfo(np.int32).max - 1
        epochs = np.iinfo(np.int32).max - 1 if num_samples is not None else 1
        self.sample_index = helpers.build_mapping(docs, sizes, epochs, n, config.sequence_length - extra_tokens,
                                                  config.short_sequence_probability, config.random_seed, min_sentences)

    def __len__(self):
        return self.sample_index.shape[0]

    def _sentences(self, idx) -> Tuple[List[List[int]], int, np.random.RandomState]:
        begin, end, target = (int(v) for v in self.sample_index[idx])
        rng = np.random.RandomState((self.config.random_seed + idx) % 2 ** 32)
        return [self.dataset[i].tolist() for i in range(begin, end)], target, rng

    def _mask(self, tokens: List[int], rng, protected: Tuple[int, ...]):
        """Returns (masked tokens, positions, original labels at those positions, spans)."""
        cfg = self.config
        cand = [i for i, t in enumerate(tokens) if t not in protected]
        budget = max(1, int(round(len(cand) * cfg.masking_probability)))
        out = list(tokens)
        rng.shuffle(cand)
        covered, spans = set(), []
        ngrams = np.arange(1, cfg.masking_max_ngram + 1)
        pv = 1.0 / ngrams
        if cfg.masking_use_longer_ngrams:
            pv = pv[::-1]
        pv = pv / pv.sum()
        for start in cand:
            if len(covered) >= budget:
                break
            if start in covered:
                continue
            n = int(rng.geometric(0.2)) if cfg.masking_use_geometric_distribution else int(rng.choice(ngrams, p=pv))
            n = min(n, cfg.masking_max_ngram, budget - len(covered))
            span = [i for i in range(start, min(start + n, len(tokens))) if tokens[i] not in protected and i not in covered]
            if not span:
                continue
            spans.append((span, [tokens[i] for i in span]))
            for i in span:
                covered.add(i)
                r = rng.random_sample()
                if r < 0.8:
                    out[i] = self.mask
                elif r < 0.9:
                    out[i] = int(rng.randint(0, self.vocab_size))
        pos = sorted(covered)
        return out, pos, [tokens[i] for i in pos], sorted(spans, key=lambda s: s[0][0])


class BERTMaskedWordPieceDataset(MaskedWordPieceDataset):
    def __init__(self, indexed_dataset, indexed_indices, num_samples, index_split, config):
        super().__init__(indexed_dataset, indexed_indices, num_samples, index_split, config,
                         min_sentences=2 if config.classification_head else 1, extra_tokens=3)

    def __getitem__(self, idx):
        sents, target, rng = self._sentences(idx)
        cfg = self.config
        if cfg.classification_head and len(sents) > 1:
            pivot = 1 if len(sents) == 2 else int(rng.randint(1, len(sents)))
            a = [t for s in sents[:pivot] for t in s]
            b = [t for s in sents[pivot:] for t in s]
            is_random = int(rng.random_sample() < 0.5)
            if is_random:
                a, b = b, a
        else:
            a, b, is_random = [t for s in sents for t in s], [], 0
        while len(a) + len(b) > target:                       # truncate the longer side, front or back at random
            side = a if len(a) > len(b) else b
            if rng.random_sample() < 0.5:
                del side[0]
            else:
                side.pop()
        tokens = [self.cls] + a + [self.sep] + (b + [self.sep] if b else [])
        types = [0] * (len(a) + 2) + [1] * (len(b) + 1 if b else 0)
        masked, pos, labels, _ = self._mask(tokens, rng, (self.cls, self.sep))
        L = cfg.sequence_length
        n = len(tokens)
        text = np.full(L, self.pad, dtype=np.int64); text[:n] = masked
        tt = np.zeros(L, dtype=np.int64); tt[:n] = types
        lab = np.full(L, -1, dtype=np.int64); lm = np.zeros(L, dtype=np.int64)
        lab[pos] = labels; lm[pos] = 1
        pm = np.zeros(L, dtype=np.int64); pm[:n] = 1
        return {"text": text, "types": tt, "labels": lab, "is_random": is_random, "padding_mask": pm,
                "loss_mask": lm, "truncated": int(n >= L)}


class T5MaskedWordPieceDataset(MaskedWordPieceDataset):
    """Masked spans are replaced by sentinel tokens in the encoder input; the decoder predicts
    sentinel + span for each."""

    def __init__(self, indexed_dataset, indexed_indices, num_samples, index_split, config):
        super().__init__(indexed_dataset, indexed_indices, num_samples, index_split, config, min_sentences=1,
                         extra_tokens=2)
        tok = config.tokenizer
        self.sentinels = list(getattr(tok, "additional_special_tokens_ids", []))
        if not self.sentinels:
            raise ValueError("the T5 dataset needs sentinel tokens (--vocab-extra-ids)")
        self.bos, self.eos = getattr(tok, "bos", tok.cls), getattr(tok, "eos", tok.sep)

    def __getitem__(self, idx):
        sents, target, rng = self._sentences(idx)
        cfg = self.config
        tokens = [t for s in sents for t in s][:target]
        _, _, _, spans = self._mask(tokens, rng, ())
        enc, dec_in, dec_out = [], [self.bos], []
        cursor = 0
        for (span, orig), sentinel in zip(spans, self.sentinels):
            enc.extend(tokens[cursor:span[0]])
            enc.append(sentinel)
            dec_in.append(sentinel); dec_in.extend(orig)
            dec_out.append(sentinel); dec_out.extend(orig)
            cursor = span[-1] + 1
        enc.extend(tokens[cursor:])
        dec_out.append(self.eos)
        Le = cfg.sequence_length_encoder or cfg.sequence_length
        Ld = cfg.sequence_length_decoder or cfg.sequence_length
        enc, dec_in, dec_out = enc[:Le], dec_in[:Ld], dec_out[:Ld]
        e = np.full(Le, self.pad, dtype=np.int64); e[:len(enc)] = enc
        d = np.full(Ld, self.pad, dtype=np.int64); d[:len(dec_in)] = dec_in
        lab = np.full(Ld, -1, dtype=np.int64); lab[:len(dec_out)] = dec_out
        lm = (lab != -1).astype(np.int64)
        em, dm = (e != self.pad).astype(np.int64), (d != self.pad).astype(np.int64)
        return {"text_enc": e, "text_dec": d, "labels": lab, "loss_mask": lm, "truncated": int(len(tokens) >= target),
                "enc_mask": em, "dec_mask": dm}
