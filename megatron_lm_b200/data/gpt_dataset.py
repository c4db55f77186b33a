"""GPT pre-training datasets: packed samples over an indexed corpus, a mock corpus, blending and
the train/valid/test builder.

Sample construction follows the reference so that a given (corpus, seed, sequence length) yields
the same samples (megatron/core/datasets/gpt_dataset.py:66-700): documents are tiled ``num_epochs``
times and shuffled (the last epoch separately when it is a small remainder, :558-590); the C++
helper maps sample -> (document position, offset) for ``seq_length + 1`` token windows crossing
document boundaries (helpers.cpp:142-247); a shuffle index permutes samples (:592-622); indices are
cached on disk keyed by an MD5 of the configuration; ``tokens = sample[:-1]``,
``labels = sample[1:]``, the loss mask zeroes EOD (optional) and padding, position ids and the
attention mask can reset at EOD (:624-700).  The mock corpus is 100 000 sequences of lengths
``default_rng(0).integers(1, 4096)``, each ``arange(1, len)`` followed by EOD (:701-750).
"""
from __future__ import annotations

import hashlib
import json
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Type

import numpy as np
import torch

from . import helpers
from .indexed_dataset import IndexedDataset


@dataclass
class BlendedMegatronDatasetConfig:
    random_seed: int = 1234
    sequence_length: int = 1024
    blend: Optional[Tuple[List[str], Optional[List[float]]]] = None
    blend_per_split: Optional[List[Optional[Tuple[List[str], Optional[List[float]]]]]] = None
    split: Optional[str] = None
    split_matrix: Optional[List[Optional[Tuple[float, float]]]] = None
    num_dataset_builder_threads: int = 1
    path_to_cache: Optional[str] = None
    mmap_bin_files: bool = True
    mock: bool = False
    tokenizer: object = None
    mid_level_dataset_surplus: float = 0.005

    def __post_init__(self):
        if self.blend_per_split is not None and any(b is not None for b in self.blend_per_split):
            if self.blend is not None:
                raise ValueError("blend and blend_per_split are mutually exclusive")
            if len(self.blend_per_split) != 3:
                raise ValueError("blend_per_split needs train/valid/test entries")
        elif self.blend is None and not self.mock:
            self.mock = True
        if self.split is not None:
            self.split_matrix = convert_split_vector_to_split_matrix(parse_and_normalize_split(self.split))
        elif self.split_matrix is None and self.blend_per_split is None:
            self.split = "1,0,0"
            self.split_matrix = convert_split_vector_to_split_matrix([1.0, 0.0, 0.0])


@dataclass
class GPTDatasetConfig(BlendedMegatronDatasetConfig):
    reset_position_ids: bool = False
    reset_attention_mask: bool = False
    eod_mask_loss: bool = False
    create_attention_mask: bool = True
    drop_last_partial_validation_sequence: bool = True
    add_extra_token_to_sequence: bool = True
    object_storage_cache_path: Optional[str] = None


def parse_and_normalize_split(split: str) -> List[float]:
    parts = [float(x) for x in split.replace("/", ",").split(",")]
    parts = (parts + [0.0] * 3)[:3]
    tot = sum(parts)
    if tot <= 0 or any(p < 0 for p in parts):
        raise ValueError(f"bad split {split!r}")
    return [p / tot for p in parts]


def convert_split_vector_to_split_matrix(vec: Sequence[float]) -> List[Optional[Tuple[float, float]]]:
    out, acc = [], 0.0
    for v in vec:
        out.append((acc, acc + v) if v > 0 else None)
        acc += v
    return out


# ----------------------------------------------------------------------------- low level
class MockGPTLowLevelDataset:
    seed: int = 0
    size: int = 100000
    max_sequence_length: int = 4096

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer
        rng = np.random.default_rng(seed=self.seed)
        self.sequence_lengths = rng.integers(low=1, high=self.max_sequence_length, size=self.size, dtype=np.int32)

    def __len__(self):
        return self.size

    def __getitem__(self, idx: int) -> np.ndarray:
        n = int(self.sequence_lengths[idx])
        return np.concatenate([np.arange(n - 1) + 1, np.array([self.tokenizer.eod])]).astype(np.int64)

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        if length is None:
            length = int(self.sequence_lengths[idx]) - offset
        return self[idx][offset:offset + length]


def _hash_config(d: dict) -> str:
    return hashlib.md5(json.dumps(d, indent=4, sort_keys=True, default=str).encode("utf-8")).hexdigest()


class GPTDataset(torch.utils.data.Dataset):
    def __init__(self, low_level, dataset_path: Optional[str], indexed_indices: np.ndarray, num_samples: Optional[int],
                 index_split: str, config: GPTDatasetConfig):
        self.dataset, self.dataset_path, self.indices = low_level, dataset_path, indexed_indices
        self.num_samples, self.index_split, self.config = num_samples, index_split, config
        self.unique_identifiers = dict(cls=type(self).__name__, dataset_path=dataset_path, num_samples=num_samples,
                                       index_split=index_split, random_seed=config.random_seed,
                                       sequence_length=config.sequence_length, split=config.split,
                                       add_extra_token=config.add_extra_token_to_sequence,
                                       n_docs=int(len(indexed_indices)))
        self.unique_description_hash = _hash_config(self.unique_identifiers)
        tok = config.tokenizer
        self._pad_token_id = getattr(tok, "pad", None)
        if self._pad_token_id is None:
            self._pad_token_id = -1
        self.eod = tok.eod
        self.masks_cacheable = not any([config.reset_position_ids, config.reset_attention_mask, config.eod_mask_loss])
        self._cached = None
        self.document_index, self.sample_index, self.shuffle_index = self._build_indices()

    # -- index construction ----------------------------------------------------
    def _num_tokens_per_epoch(self) -> int:
        return int(np.sum(self.dataset.sequence_lengths[self.indices]))

    def _num_epochs(self, tokens_per_epoch: int) -> int:
        if self.num_samples is None:
            return 1
        extra = int(self.config.add_extra_token_to_sequence)
        epochs, tokens = 0, 0
        need = self.num_samples * self.config.sequence_length + extra
        while tokens < need:
            epochs += 1
            tokens += tokens_per_epoch
        return max(epochs, 1)

    def _build_indices(self):
        cfg = self.config
        cache = cfg.path_to_cache
        paths = None
        if cache is not None:
            base = os.path.join(cache, f"{self.unique_description_hash}-{type(self).__name__}-{self.index_split}")
            paths = [base + s for s in ("-document_index.npy", "-sample_index.npy", "-shuffle_index.npy")]
            if all(os.path.isfile(p) for p in paths):
                return tuple(np.load(p, allow_pickle=True, mmap_mode="r") for p in paths)
        rng = np.random.RandomState(cfg.random_seed)
        tokens_per_epoch = self._num_tokens_per_epoch()
        num_epochs = self._num_epochs(tokens_per_epoch)
        extra = int(cfg.add_extra_token_to_sequence)
        if num_epochs == 1:
            separate_final_epoch = False
        else:
            per_epoch = (tokens_per_epoch - extra) // cfg.sequence_length
            from_prev = ((num_epochs - 1) * tokens_per_epoch - extra) // cfg.sequence_length
            last = self.num_samples - from_prev
            separate_final_epoch = last < int(0.80 * per_epoch)
        document_index = _build_document_index(self.indices, num_epochs, rng, separate_final_epoch)
        drop_last = True
        if self.index_split == "valid":
            drop_last = cfg.drop_last_partial_validation_sequence
        sample_index = helpers.build_sample_idx(self.dataset.sequence_lengths, document_index, cfg.sequence_length,
                                                num_epochs, tokens_per_epoch, drop_last, extra)
        n = sample_index.shape[0] - 1
        if separate_final_epoch:
            first = ((num_epochs - 1) * tokens_per_epoch - extra) // cfg.sequence_length
            shuffle_index = _build_shuffle_index(first, n, rng)
        else:
            shuffle_index = _build_shuffle_index(n, n, rng)
        if paths is not None and (not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0):
            os.makedirs(cache, exist_ok=True)
            with open(os.path.join(cache, f"{self.unique_description_hash}-{type(self).__name__}-{self.index_split}"
                                   "-description.txt"), "w") as f:
                json.dump(self.unique_identifiers, f, indent=4, default=str)
            for p, a in zip(paths, (document_index, sample_index, shuffle_index)):
                np.save(p, a, allow_pickle=True)
        return document_index, sample_index, shuffle_index

    def __len__(self) -> int:
        return self.sample_index.shape[0] - 1

    # -- sample assembly ---------------------------------------------------------
    def _tokens(self, idx: int) -> Tuple[np.ndarray, np.ndarray]:
        idx = int(self.shuffle_index[idx])
        d0, o0 = self.sample_index[idx]
        d1, o1 = self.sample_index[idx + 1]
        extra = int(self.config.add_extra_token_to_sequence)
        docs, parts = [], []
        if d0 == d1:
            docs.append(self.document_index[d0])
            parts.append(self.dataset.get(int(self.document_index[d0]), offset=int(o0), length=int(o1 - o0 + extra)))
        else:
            for i in range(int(d0), int(d1) + 1):
                docs.append(self.document_index[i])
                off = int(o0) if i == d0 else 0
                length = None if i < d1 else int(o1) + extra
                parts.append(self.dataset.get(int(self.document_index[i]), offset=off, length=length))
        tokens = np.concatenate(parts).astype(np.int64)
        want = self.config.sequence_length + extra
        if len(tokens) < want:
            tokens = np.concatenate([tokens, np.full(want - len(tokens), self._pad_token_id, dtype=np.int64)])
        return tokens, np.asarray(docs, dtype=np.int64)

    def __getitem__(self, idx: Optional[int]) -> Dict[str, torch.Tensor]:
        if idx is None:
            text = np.full(self.config.sequence_length + 1, self._pad_token_id, dtype=np.int64)
        else:
            text, _ = self._tokens(idx)
        text = torch.from_numpy(text).long()
        if self.config.add_extra_token_to_sequence:
            tokens, labels = text[:-1].contiguous(), text[1:].contiguous()
        else:
            tokens = text
            labels = torch.roll(text, shifts=-1, dims=0)
            labels[-1] = self._pad_token_id
        if not self.masks_cacheable or self._cached is None:
            am, lm, pos = get_ltor_masks_and_position_ids(tokens, self.eod, self.config.reset_position_ids,
                                                          self.config.reset_attention_mask, self.config.eod_mask_loss,
                                                          self.config.create_attention_mask)
            if self.masks_cacheable:
                self._cached = (am, lm, pos)
        else:
            am, lm, pos = self._cached
        lm = lm.clone()
        lm[labels == self._pad_token_id] = 0.0
        tokens = tokens.clone()
        labels = labels.clone()
        tokens[tokens == self._pad_token_id] = 0
        labels[labels == self._pad_token_id] = 0
        if idx is None:
            lm = torch.zeros_like(lm)
        out = {"tokens": tokens, "labels": labels, "loss_mask": lm, "position_ids": pos}
        if self.config.create_attention_mask:
            out["attention_mask"] = am
        return out


class MockGPTDataset(GPTDataset):
    pass


def _build_document_index(documents: np.ndarray, num_epochs: int, rng: np.random.RandomState,
                          separate_final_epoch: bool) -> np.ndarray:
    if not separate_final_epoch or num_epochs == 1:
        idx = np.tile(np.asarray(documents, dtype=np.int32), num_epochs)
        rng.shuffle(idx)
        return idx
    first = _build_document_index(documents, num_epochs - 1, rng, False)
    last = _build_document_index(documents, 1, rng, False)
    return np.concatenate((first, last))


def _build_shuffle_index(num_samples: int, total_size: int, rng: np.random.RandomState) -> np.ndarray:
    dtype = np.uint32 if total_size < (np.iinfo(np.uint32).max - 1) else np.int64
    first = np.arange(0, num_samples, dtype=dtype)
    rng.shuffle(first)
    if num_samples == total_size:
        return first
    last = np.arange(num_samples, total_size, dtype=dtype)
    rng.shuffle(last)
    return np.concatenate((first, last))


def get_ltor_masks_and_position_ids(data: torch.Tensor, eod_token: int, reset_position_ids: bool,
                                    reset_attention_mask: bool, eod_mask_loss: bool, create_attention_mask: bool):
    """Left-to-right masks and position ids for one sequence (reference: gpt_dataset.py:624-700)."""
    n = data.numel()
    am = torch.tril(torch.ones((n, n))).unsqueeze(0) if create_attention_mask else None
    lm = torch.ones(n, dtype=torch.float)
    if eod_mask_loss:
        lm[data == eod_token] = 0.0
    pos = torch.arange(n, dtype=torch.long)
    if reset_position_ids or reset_attention_mask:
        eods = pos[data == eod_token]
        prev = 0
        for j in range(eods.numel()):
            i = int(eods[j])
            if reset_attention_mask and am is not None:
                am[0, (i + 1):, :(i + 1)] = 0
            if reset_position_ids:
                pos[(i + 1):] -= i + 1 - prev
                prev = i + 1
    if am is not None:
        am = am < 0.5
    return am, lm, pos


# ----------------------------------------------------------------------------- blending
class BlendedDataset(torch.utils.data.Dataset):
    """Interleaves datasets in proportion to ``weights`` (or exhaustively when ``size`` is None)
    (reference: blended_dataset.py:24)."""

    def __init__(self, datasets: Sequence[torch.utils.data.Dataset], weights: Sequence[float], size: Optional[int],
                 config: BlendedMegatronDatasetConfig):
        if len(datasets) != len(weights) or len(datasets) >= 32767:
            raise ValueError("datasets and weights must match (and be fewer than 32767)")
        self.datasets, self.config = list(datasets), config
        w = np.asarray(weights, dtype=np.float64)
        self.weights = (w / w.sum()).tolist()
        self.size = size
        if size is None:
            self.dataset_index, self.dataset_sample_index = helpers.build_exhaustive_blending_indices(
                [len(d) for d in datasets])
        else:
            self.dataset_index, self.dataset_sample_index = helpers.build_blending_indices(self.weights, size)
            for d, ds in enumerate(self.datasets):
                need = int(self.dataset_sample_index[self.dataset_index == d].max(initial=-1)) + 1
                if need > len(ds):
                    raise IndexError(f"blend asks dataset {d} for {need} samples but it has {len(ds)}")

    def __len__(self) -> int:
        return len(self.dataset_index)

    def __getitem__(self, idx: int):
        d = int(self.dataset_index[idx])
        return {"dataset_id": d, **self.datasets[d][int(self.dataset_sample_index[idx])]}


class BlendedMegatronDatasetBuilder:
    """Builds the (train, valid, test) datasets for a blend (reference:
    blended_megatron_dataset_builder.py:28)."""

    def __init__(self, cls: Type[GPTDataset], sizes: Sequence[Optional[int]], is_built_on_rank: Callable[[], bool],
                 config: GPTDatasetConfig):
        self.cls, self.sizes, self.is_built_on_rank, self.config = cls, list(sizes), is_built_on_rank, config

    def _low_level(self, prefix: Optional[str]):
        if self.config.mock or prefix is None:
            return MockGPTLowLevelDataset(self.config.tokenizer)
        osc = None
        cache = getattr(self.config, "object_storage_cache_path", None)
        if cache:
            from .object_storage import ObjectStorageConfig
            osc = ObjectStorageConfig(path_to_idx_cache=cache)
        return IndexedDataset(prefix, mmap=self.config.mmap_bin_files, object_storage_config=osc)

    def _split_one(self, prefix: Optional[str], sizes: Sequence[Optional[int]], split_matrix) -> List[Optional[GPTDataset]]:
        low = self._low_level(prefix)
        n_docs = len(low.document_indices) - 1 if hasattr(low, "document_indices") else len(low)
        out = []
        for i, name in enumerate(("train", "valid", "test")):
            rng_ = split_matrix[i] if split_matrix is not None else None
            if rng_ is None or not self.is_built_on_rank():
                out.append(None)
                continue
            lo, hi = int(round(rng_[0] * n_docs)), int(round(rng_[1] * n_docs))
            if hi <= lo:
                out.append(None)
                continue
            docs = np.arange(lo, hi, dtype=np.int32)
            out.append(self.cls(low, prefix, docs, sizes[i], name, self.config))
        return out

    def build(self) -> List[Optional[torch.utils.data.Dataset]]:
        cfg = self.config
        if cfg.mock or (cfg.blend is None and cfg.blend_per_split is None):
            return self._split_one(None, self.sizes, cfg.split_matrix)
        if cfg.blend is not None:
            prefixes, weights = cfg.blend
            if len(prefixes) == 1:
                return self._split_one(prefixes[0], self.sizes, cfg.split_matrix)
            w = np.asarray(weights if weights is not None else [1.0] * len(prefixes), dtype=np.float64)
            w = w / w.sum()
            per = [[None if s is None else int(np.ceil(s * wi * (1 + cfg.mid_level_dataset_surplus))) for s in self.sizes]
                   for wi in w]
            parts = [self._split_one(p, sz, cfg.split_matrix) for p, sz in zip(prefixes, per)]
            out = []
            for i in range(3):
                ds = [p[i] for p in parts]
                if any(d is None for d in ds):
                    out.append(None)
                else:
                    out.append(BlendedDataset(ds, w.tolist(), self.sizes[i], cfg))
            return out
        out = []
        for i, blend in enumerate(cfg.blend_per_split):
            if blend is None:
                out.append(None)
                continue
            prefixes, weights = blend
            matrix = [None, None, None]
            matrix[i] = (0.0, 1.0)
            sizes = [None, None, None]
            sizes[i] = self.sizes[i]
            ds = [self._split_one(p, sizes, matrix)[i] for p in prefixes]
            if len(ds) == 1:
                out.append(ds[0])
            else:
                w = weights if weights is not None else [1.0] * len(ds)
                out.append(BlendedDataset(ds, w, self.sizes[i], cfg))
        return out


# ----------------------------------------------------------------------------- samplers
class MegatronPretrainingSampler:
    """Sequential batches from ``consumed_samples`` on, strided over data-parallel ranks
    (reference: megatron/legacy/data/data_samplers.py)."""

    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, data_parallel_rank: int,
                 data_parallel_size: int, drop_last: bool = True):
        if total_samples <= 0 or consumed_samples >= total_samples or micro_batch_size <= 0:
            raise ValueError("bad sampler sizes")
        if data_parallel_rank >= data_parallel_size:
            raise ValueError("data_parallel_rank out of range")
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size, self.drop_last = micro_batch_size, drop_last
        self.dp_rank, self.dp_size = data_parallel_rank, data_parallel_size
        self.global_micro = micro_batch_size * data_parallel_size

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        batch = []
        for idx in range(self.consumed_samples, self.total_samples):
            batch.append(idx)
            if len(batch) == self.global_micro:
                s = self.dp_rank * self.micro_batch_size
                yield batch[s:s + self.micro_batch_size]
                batch = []
        if batch and not self.drop_last:
            s = self.dp_rank * self.micro_batch_size
            yield batch[s:s + self.micro_batch_size]


class MegatronPretrainingRandomSampler:
    """Epoch-wise shuffled batches, resumable from ``consumed_samples``."""

    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int, data_parallel_rank: int,
                 data_parallel_size: int, seed: int = 1234):
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size = micro_batch_size
        self.dp_rank, self.dp_size = data_parallel_rank, data_parallel_size
        self.global_micro = micro_batch_size * data_parallel_size
        self.last_batch_size = total_samples % self.global_micro
        self.seed = seed

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        active = self.total_samples - self.last_batch_size
        epoch = self.consumed_samples // active
        current = self.consumed_samples % active
        bucket = (self.total_samples // self.global_micro) * self.micro_batch_size
        offset = current // self.dp_size
        start = self.dp_rank * bucket
        g = torch.Generator()
        g.manual_seed(self.seed + epoch)
        order = (start + torch.randperm(bucket, generator=g)).tolist()[offset:]
        batch = []
        for idx in order:
            batch.append(idx)
            if len(batch) == self.micro_batch_size:
                self.consumed_samples += self.global_micro
                yield batch
                batch = []


def build_pretraining_data_loader(dataset, consumed_samples: int, micro_batch_size: int, dp_rank: int, dp_size: int,
                                  dataloader_type: str = "single", num_workers: int = 0, seed: int = 1234):
    if dataset is None:
        return None
    if dataloader_type == "single":
        sampler = MegatronPretrainingSampler(len(dataset), consumed_samples, micro_batch_size, dp_rank, dp_size)
    elif dataloader_type == "cyclic":
        sampler = MegatronPretrainingRandomSampler(len(dataset), consumed_samples, micro_batch_size, dp_rank, dp_size,
                                                   seed)
    else:
        raise ValueError(f"unknown dataloader type {dataloader_type}")
    return torch.utils.data.DataLoader(dataset, batch_sampler=sampler, num_workers=num_workers, pin_memory=True,
                                       persistent_workers=num_workers > 0)
