"""Text + image pairs into one multimodal indexed dataset (reference: tools/preprocess_mmdata.py).

Every document is two sequences: the caption's token ids (mode 0), padded with the end-of-document id to
``--pad-length`` when ``--append-eod`` is given, and the image file's bytes (mode 1) packed four to an int32 word,
with the count of zero bytes added at the end stored in front.  ``decode_image_bytes`` undoes the packing.

    python -m megatron_lm_b200.data.preprocess_mmdata --input captions.jsonl --input-image images/ \\
        --output-prefix out --tokenizer-type GPT2BPETokenizer --vocab-file ... --merge-file ... --pad-length 64
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

from .indexed_dataset import IndexedDatasetBuilder, get_bin_path, get_idx_path
from .tokenizer import build_tokenizer

TEXT_MODE, IMAGE_MODE = 0, 1


def encode_image_bytes(raw: bytes) -> np.ndarray:
    pad = (4 - len(raw) % 4) % 4
    words = np.frombuffer(raw + b"\0" * pad, dtype=np.int32)
    return np.concatenate((np.asarray([pad], dtype=np.int32), words))


def decode_image_bytes(seq: np.ndarray) -> bytes:
    pad = int(seq[0])
    raw = np.ascontiguousarray(seq[1:], dtype=np.int32).tobytes()
    return raw[:len(raw) - pad] if pad else raw


def main(argv=None):
    ap = argparse.ArgumentParser(description="Build a multimodal (text, image) indexed dataset.")
    ap.add_argument("--input", required=True, help="JSON-lines file with a 'text' field per record")
    ap.add_argument("--input-image", required=True, help="directory of image files, paired with the records in "
                                                         "sorted file-name order")
    ap.add_argument("--pad-length", type=int, required=True)
    ap.add_argument("--tokenizer-type", required=True)
    ap.add_argument("--tokenizer-model", default=None)
    ap.add_argument("--vocab-file", default=None)
    ap.add_argument("--merge-file", default=None)
    ap.add_argument("--vocab-size", type=int, default=None)
    ap.add_argument("--append-eod", action="store_true")
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--log-interval", type=int, default=100)
    a = ap.parse_args(argv)
    a.rank, a.make_vocab_size_divisible_by, a.tensor_model_parallel_size, a.vocab_extra_ids = 0, 128, 1, 0
    tok = build_tokenizer(a)
    images = sorted(os.path.join(a.input_image, f) for f in os.listdir(a.input_image))
    b = IndexedDatasetBuilder(get_bin_path(a.output_prefix), dtype=np.int32, multimodal=True)
    t0, n = time.time(), 0
    with open(a.input, "r", encoding="utf-8") as fin:
        for n, (line, img) in enumerate(zip(fin, images), 1):
            ids = list(tok.tokenize(json.loads(line)["text"]))
            if ids and a.append_eod:
                ids = ids[:a.pad_length]
                ids += [tok.eod] * (a.pad_length - len(ids))
            with open(img, "rb") as f:
                words = encode_image_bytes(f.read())
            b.add_item(np.asarray(ids, dtype=np.int32), TEXT_MODE)
            b.add_item(words, IMAGE_MODE)
            b.end_document()
            if n % a.log_interval == 0:
                print(f"processed {n} documents ({n / (time.time() - t0):.1f} docs/s)", file=sys.stderr)
    b.finalize(get_idx_path(a.output_prefix))
    print(f"{n} documents -> {a.output_prefix}.bin/.idx")


if __name__ == "__main__":
    main()
