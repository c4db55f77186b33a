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


def test_indexed_dataset_from_an_object_store(tmp_path):
    """``s3://`` prefixes: the index is cached locally once, tokens come through ranged reads served from a chunk
    cache (reference: tests/unit_tests/data/test_preprocess_data.py object-storage readers with a mock client)."""
    from megatron_lm_b200.data import object_storage as osu
    rng = np.random.default_rng(3)
    docs = [rng.integers(0, 1000, rng.integers(5, 60)) for _ in range(40)]
    root = tmp_path / "store"
    (root / "corpora").mkdir(parents=True)
    _write_corpus(str(root / "corpora" / "wiki"), docs)
    client = osu.LocalDirectoryClient(str(root))
    osu.register_client_factory("s3", lambda: client)
    try:
        prefix = "s3://corpora/wiki"
        assert osu.is_object_storage_path(prefix) and not osu.is_object_storage_path("/data/wiki")
        assert osu.parse_s3_path("s3://corpora/a/b.bin") == ("corpora", "a/b.bin")
        assert osu.get_object_storage_access("msc://p/x") == "msc"
        with pytest.raises(ValueError):
            osu.parse_s3_path("/local/file")
        assert IndexedDataset.exists(prefix) and not IndexedDataset.exists("s3://corpora/missing")
        with pytest.raises(ValueError):
            IndexedDataset(prefix)                                               # no cache configuration
        cfg = osu.ObjectStorageConfig(path_to_idx_cache=str(tmp_path / "idx_cache"), bin_chunk_nbytes=256)
        ds = IndexedDataset(prefix, object_storage_config=cfg)
        assert os.path.isfile(osu.get_index_cache_path(prefix + ".idx", cfg))
        assert len(ds) == 40
        before = client.requests
        for i in range(40):
            assert np.array_equal(ds[i], docs[i])
        used = client.requests - before
        total_bytes = sum(len(d) for d in docs) * 2
        assert used <= total_bytes // 256 + 2, (used, total_bytes)               # sequential reads: one per chunk
        assert np.array_equal(ds.get(7, 2, 3), docs[7][2:5])
        assert all(np.array_equal(a, b) for a, b in zip(ds[3:9], docs[3:9]))       # a slice larger than one chunk
        # a second open finds the cached index: no download
        before = client.requests
        IndexedDataset(prefix, object_storage_config=cfg)
        assert client.requests == before
        # the GPT dataset builder reaches the store through its configuration
        gcfg = GPTDatasetConfig(random_seed=1, sequence_length=8, blend=([prefix], None), split="1,0,0",
                                tokenizer=NullTokenizer(999), path_to_cache=str(tmp_path / "cache"),
                                object_storage_cache_path=str(tmp_path / "idx_cache"), mmap_bin_files=False)
        train, _, _ = BlendedMegatronDatasetBuilder(GPTDataset, [20, None, None], lambda: True, gcfg).build()
        assert train[0]["tokens"].shape == (8,)
    finally:
        osu.register_client_factory("s3", osu._boto3_client)


def test_mock_multimodal_dataset():
    from megatron_lm_b200.data.multimodal_dataset import MockMultimodalDataset, MultimodalDatasetConfig
    with pytest.raises(ValueError):
        MultimodalDatasetConfig(sequence_length=16, tokenizer=NullTokenizer(99), mock=True, image_h=8, image_w=8)
    seen = []

    def prep(sample):
        seen.append(set(sample))
        sample["tokens"] = torch.cat([torch.full((2,), -200), sample["tokens"]])      # image placeholder tokens
        return sample
    cfg = MultimodalDatasetConfig(random_seed=5, sequence_length=16, tokenizer=NullTokenizer(99), mock=True, image_h=8,
                                  image_w=12, preprocess_func=prep, split="1,0,0")
    train, _, _ = BlendedMegatronDatasetBuilder(MockMultimodalDataset, [10, None, None], lambda: True, cfg).build()
    a, b = train[0], train[0]
    assert a["image"].shape == (3, 8, 12) and 0 <= float(a["image"].min()) and float(a["image"].max()) < 1
    assert torch.equal(a["image"], b["image"]) and not torch.equal(a["image"], train[1]["image"])
    assert a["tokens"].shape == (18,) and "image" in seen[0] and "labels" in seen[0]
