"""Indexed dataset format, GPT sample construction, blending, samplers, tokenizers."""
import json
import os

import numpy as np
import pytest
import torch

from megatron_lm_b200.data.gpt_dataset import (BlendedMegatronDatasetBuilder, GPTDataset, GPTDatasetConfig,
                                               MegatronPretrainingSampler, MockGPTDataset,
                                               get_ltor_masks_and_position_ids)
from megatron_lm_b200.data.indexed_dataset import IndexedDataset, IndexedDatasetBuilder, optimal_dtype
from megatron_lm_b200.data.tokenizer import (GPT2BPETokenizer, NullTokenizer, build_tokenizer,
                                             vocab_size_with_padding)


def _write_corpus(prefix, docs, dtype=np.uint16):
    b = IndexedDatasetBuilder(prefix + ".bin", dtype=dtype)
    for d in docs:
        b.add_item(d)
        b.end_document()
    b.finalize(prefix + ".idx")


def test_indexed_dataset_roundtrip(tmp_path):
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 1000, rng.integers(1, 50)) for _ in range(37)]
    prefix = str(tmp_path / "c")
    _write_corpus(prefix, docs)
    for mmap in (True, False):
        ds = IndexedDataset(prefix, mmap=mmap)
        assert len(ds) == 37 and ds.index.dtype == np.uint16
        for i in (0, 5, 36):
            assert np.array_equal(ds[i], docs[i])
        assert np.array_equal(ds.get(7, 2, 3), docs[7][2:5]) or len(docs[7]) < 5
        sl = ds[3:6]
        assert all(np.array_equal(a, b) for a, b in zip(sl, docs[3:6]))
    with open(prefix + ".idx", "rb") as f:
        assert f.read(9) == b"MMIDIDX\x00\x00"
    assert optimal_dtype(50000) == np.uint16 and optimal_dtype(70000) == np.int32


def test_gpt_dataset_samples_tile_the_token_stream(tmp_path):
    rng = np.random.default_rng(1)
    docs = [np.concatenate([rng.integers(1, 500, rng.integers(3, 40)), [0]]) for _ in range(60)]
    prefix = str(tmp_path / "c")
    _write_corpus(prefix, docs)
    cfg = GPTDatasetConfig(random_seed=7, sequence_length=16, blend=([prefix], None), split="1,0,0",
                           tokenizer=NullTokenizer(499), path_to_cache=str(tmp_path / "cache"),
                           reset_position_ids=True, reset_attention_mask=True, eod_mask_loss=True)
    low = IndexedDataset(prefix)
    ds = GPTDataset(low, prefix, np.arange(60, dtype=np.int32), 100, "train", cfg)
    assert len(ds) >= 100
    s = ds[0]
    assert s["tokens"].shape == (16,) and s["labels"].shape == (16,)
    assert torch.equal(s["tokens"][1:], s["labels"][:-1])
    # un-shuffled order reproduces the concatenated (shuffled-document) token stream
    stream = np.concatenate([docs[d] for d in ds.document_index])
    inv = np.argsort(ds.shuffle_index)
    for k in range(5):
        tok, _ = ds._tokens(int(inv[k]))
        assert np.array_equal(tok, stream[k * 16:k * 16 + 17])
    ds2 = GPTDataset(low, prefix, np.arange(60, dtype=np.int32), 100, "train", cfg)     # from the cache
    assert np.array_equal(ds2.shuffle_index, ds.shuffle_index)


def test_masks_and_position_reset():
    data = torch.tensor([5, 6, 0, 7, 8, 9, 0, 4])
    am, lm, pos = get_ltor_masks_and_position_ids(data, 0, True, True, True, True)
    assert pos.tolist() == [0, 1, 2, 0, 1, 2, 3, 0]
    assert lm.tolist() == [1, 1, 0, 1, 1, 1, 0, 1]
    assert bool(am[0, 4, 1]) and not bool(am[0, 4, 3])          # True = masked out


def test_mock_dataset_and_builder():
    cfg = GPTDatasetConfig(random_seed=0, sequence_length=64, mock=True, split="969,30,1", tokenizer=NullTokenizer(64))
    train, valid, test = BlendedMegatronDatasetBuilder(MockGPTDataset, [200, 20, None], lambda: True, cfg).build()
    assert len(train) >= 200 and valid is not None
    x = train[3]
    assert x["tokens"].max() < 4096 and x["loss_mask"].sum() > 0


def test_blend_of_two_corpora(tmp_path):
    rng = np.random.default_rng(2)
    prefixes = []
    for n in range(2):
        docs = [rng.integers(1, 100, 30) for _ in range(40)]
        p = str(tmp_path / f"c{n}")
        _write_corpus(p, docs)
        prefixes.append(p)
    cfg = GPTDatasetConfig(random_seed=3, sequence_length=8, blend=(prefixes, [0.75, 0.25]), split="1,0,0",
                           tokenizer=NullTokenizer(100))
    train, _, _ = BlendedMegatronDatasetBuilder(GPTDataset, [80, None, None], lambda: True, cfg).build()
    ids = [train[i]["dataset_id"] for i in range(80)]
    assert abs(ids.count(0) - 60) <= 1


def test_sampler_is_dp_strided_and_resumable():
    a = list(MegatronPretrainingSampler(20, 0, 2, 0, 2))
    b = list(MegatronPretrainingSampler(20, 0, 2, 1, 2))
    assert a[0] == [0, 1] and b[0] == [2, 3] and a[1] == [4, 5]
    resumed = list(MegatronPretrainingSampler(20, 8, 2, 0, 2))
    assert resumed[0] == [8, 9]


def test_tokenizers(tmp_path):
    t = NullTokenizer(100)
    assert t.tokenize("1 2 3") == [1, 2, 3] and t.eod == 100 and t.vocab_size == 101
    assert vocab_size_with_padding(50257, 128, 2) == 50432
    vocab = {"<|endoftext|>": 0, "h": 1, "e": 2, "l": 3, "o": 4, "he": 5, "ll": 6, "hell": 7, "hello": 8, "Ġ": 9,
             "w": 10, "Ġw": 11}
    (tmp_path / "v.json").write_text(json.dumps(vocab))
    (tmp_path / "m.txt").write_text("#version\nh e\nl l\nhe ll\nhell o\nĠ w\n")
    g = GPT2BPETokenizer(str(tmp_path / "v.json"), str(tmp_path / "m.txt"))
    assert g.tokenize("hello") == [8]
    assert g.detokenize(g.tokenize("hello w")) == "hello w"

    class A:
        tokenizer_type = "NullTokenizer"
        vocab_size = 1000
        padded_vocab_size = None
        make_vocab_size_divisible_by = 128
        tensor_model_parallel_size = 1
    args = A()
    build_tokenizer(args)
    assert args.padded_vocab_size == 1024
