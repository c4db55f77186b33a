"""preprocess_data / merge_datasets round trip, and SFT masking."""
import json
import os

import numpy as np
import torch

from megatron_lm_b200.data import merge_datasets, preprocess_data
from megatron_lm_b200.data.indexed_dataset import IndexedDataset
from megatron_lm_b200.data.sft_dataset import SFTDataset
from megatron_lm_b200.data.tokenizer import NullTokenizer


def _write(path, docs):
    with open(path, "w") as f:
        for d in docs:
            f.write(json.dumps({"text": d}) + "\n")


def test_preprocess_and_merge(tmp_path):
    docs = ["1 2 3 4", "5 6", "7 8 9 10 11"]
    src = tmp_path / "c.jsonl"
    _write(src, docs)
    out = str(tmp_path / "a")
    preprocess_data.main(["--input", str(src), "--output-prefix", out, "--tokenizer-type", "NullTokenizer",
                          "--vocab-size", "100", "--append-eod"])
    ds = IndexedDataset(out + "_text_document")
    assert len(ds) == 3
    assert ds[0].tolist() == [1, 2, 3, 4, 100] and ds[2].tolist() == [7, 8, 9, 10, 11, 100]
    # partitioned run gives the same documents (order of interleaved partitions: 0, 2 | 1)
    out2 = str(tmp_path / "b")
    preprocess_data.main(["--input", str(src), "--output-prefix", out2, "--tokenizer-type", "NullTokenizer",
                          "--vocab-size", "100", "--append-eod", "--partitions", "2"])
    ds2 = IndexedDataset(out2 + "_text_document")
    assert sorted(map(tuple, (ds2[i].tolist() for i in range(3)))) == sorted(map(tuple, (ds[i].tolist() for i in range(3))))
    # merge two datasets of a directory
    d = tmp_path / "m"
    os.makedirs(d)
    for name in ("a_text_document", "b_text_document"):
        for ext in (".bin", ".idx"):
            os.replace(str(tmp_path / (name + ext)), str(d / (name + ext)))
    merge_datasets.main(["--input", str(d), "--output-prefix", str(tmp_path / "merged")])
    assert len(IndexedDataset(str(tmp_path / "merged"))) == 6


def test_sft_masks_only_assistant(tmp_path):
    tok = NullTokenizer(1000)
    conv = [{"role": "user", "content": "1 2 3"}, {"role": "assistant", "content": "4 5"}]

    class T:
        eod, pad = 999, 0
        def tokenize(self, s): return [int(x) for x in s.split() if x.isdigit()]
    ds = SFTDataset([conv], T(), sequence_length=8, template=lambda r, c: c)
    s = ds[0]
    assert s["tokens"].tolist() == [1, 2, 3, 4, 5, 999, 0, 0]
    # labels are next tokens; only assistant tokens (4, 5) and the closing eod count
    assert s["loss_mask"].tolist() == [0, 0, 1, 1, 1, 0, 0, 0]
    assert s["labels"][2:5].tolist() == [4, 5, 999]


def test_preprocess_plain_text_lines(tmp_path):
    src = tmp_path / "sents.txt"
    src.write_text("1 2 3\n4 5\n\n6 7 8 9\n")
    out = str(tmp_path / "nmt")
    preprocess_data.main(["--input", str(src), "--output-prefix", out, "--tokenizer-type", "NullTokenizer",
                          "--vocab-size", "100", "--plain-text"])
    ds = IndexedDataset(out + "_text_document")
    assert [ds[i].tolist() for i in range(len(ds))] == [[1, 2, 3], [4, 5], [6, 7, 8, 9]]


def test_preprocess_multimodal_pairs(tmp_path):
    from megatron_lm_b200.data import preprocess_mmdata as M
    imgs = tmp_path / "img"
    imgs.mkdir()
    blobs = [bytes(range(7)), bytes(range(50, 62))]
    for i, b in enumerate(blobs):
        (imgs / f"{i:03d}.bin").write_bytes(b)
    src = tmp_path / "cap.jsonl"
    _write(src, ["1 2 3", "4 5"])
    out = str(tmp_path / "mm")
    M.main(["--input", str(src), "--input-image", str(imgs), "--output-prefix", out, "--tokenizer-type", "NullTokenizer",
            "--vocab-size", "100", "--pad-length", "5", "--append-eod"])
    ds = IndexedDataset(out, multimodal=True)
    assert len(ds) == 4
    (t0, m0), (i0, mi0), (t1, m1), (i1, mi1) = (ds[i] for i in range(4))
    assert (m0, mi0, m1, mi1) == (0, 1, 0, 1)
    assert t0.tolist() == [1, 2, 3, 100, 100] and t1.tolist() == [4, 5, 100, 100, 100]
    assert M.decode_image_bytes(i0) == blobs[0] and M.decode_image_bytes(i1) == blobs[1]
