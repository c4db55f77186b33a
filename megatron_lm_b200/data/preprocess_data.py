"""Tokenise JSON-lines text into the indexed ``.bin`` / ``.idx`` format.

``python -m megatron_lm_b200.data.preprocess_data --input corpus.jsonl --output-prefix out
   --tokenizer-type GPT2BPETokenizer --vocab-file v.json --merge-file m.txt --append-eod --workers 8``

Reference: tools/preprocess_data.py (``Encoder`` :59, ``Partition`` :106, ``main`` :288): one output pair
per JSON key (``<prefix>_<key>_document`` or ``_sentence`` with ``--split-sentences``), optional
partitioning of the input across worker groups, and a merge of the partial outputs.
"""
from __future__ import annotations

import argparse
import glob
import json
import multiprocessing
import os
import sys
import time
from types import SimpleNamespace

import numpy as np

from .indexed_dataset import IndexedDatasetBuilder, get_bin_path, get_idx_path, optimal_dtype
from .tokenizer import build_tokenizer

_ENC = None


class Encoder:
    def __init__(self, args):
        self.args = args

    def initializer(self):
        global _ENC
        _ENC = SimpleNamespace(tokenizer=build_tokenizer(self.args), splitter=self._splitter())

    def _splitter(self):
        if not self.args.split_sentences:
            return lambda text: [text]
        import re
        pat = re.compile(r"(?<=[.!?])\s+")
        keep_nl = self.args.keep_newlines
        return lambda text: [s for s in (pat.split(text) if not keep_nl else re.split(r"(?<=[.!?\n])\s*", text)) if s]

    def encode(self, line: str):
        if self.args.plain_text:
            # one sentence per line, no JSON (parallel corpora for translation; reference: tools/preprocess_data_nmt.py)
            data = {k: line.rstrip("\n") for k in self.args.json_keys}
        else:
            data = json.loads(line)
        ids, lens = {}, {}
        for key in self.args.json_keys:
            text = data[key]
            doc_ids, sent_lens = [], []
            for sent in _ENC.splitter(text):
                if not sent.strip():
                    continue
                t = _ENC.tokenizer.tokenize(sent)
                if t:
                    doc_ids.extend(t)
                    sent_lens.append(len(t))
            if doc_ids and self.args.append_eod:
                doc_ids.append(_ENC.tokenizer.eod)
                sent_lens[-1] += 1
            ids[key], lens[key] = doc_ids, sent_lens
        return ids, lens, len(line)


def process_file(args, in_path: str, out_prefix: str):
    enc = Encoder(args)
    tok = build_tokenizer(args)
    level = "sentence" if args.split_sentences else "document"
    builders = {k: IndexedDatasetBuilder(get_bin_path(f"{out_prefix}_{k}_{level}"), dtype=optimal_dtype(tok.vocab_size))
                for k in args.json_keys}
    fin = open(in_path, "r", encoding="utf-8")
    if args.workers > 1:
        pool = multiprocessing.Pool(args.workers, initializer=enc.initializer)
        it = pool.imap(enc.encode, fin, 32)
    else:
        enc.initializer()
        pool, it = None, map(enc.encode, fin)
    t0, nbytes = time.time(), 0
    for i, (ids, lens, n) in enumerate(it, 1):
        nbytes += n
        for k in args.json_keys:
            if ids[k]:
                builders[k].add_document(ids[k], lens[k])
        if i % args.log_interval == 0:
            dt = time.time() - t0
            print(f"processed {i} documents ({i / dt:.1f} docs/s, {nbytes / dt / 1e6:.2f} MB/s)", file=sys.stderr)
    if pool is not None:
        pool.close()
    fin.close()
    for k, b in builders.items():
        b.finalize(get_idx_path(f"{out_prefix}_{k}_{level}"))


def merge_partitions(args, parts, out_prefix):
    tok = build_tokenizer(args)
    level = "sentence" if args.split_sentences else "document"
    for k in args.json_keys:
        full = f"{out_prefix}_{k}_{level}"
        b = IndexedDatasetBuilder(get_bin_path(full), dtype=optimal_dtype(tok.vocab_size))
        for p in parts:
            b.add_index(f"{p}_{k}_{level}")
        b.finalize(get_idx_path(full))
        if not args.keep_sequential_samples:
            for p in parts:
                os.remove(get_bin_path(f"{p}_{k}_{level}"))
                os.remove(get_idx_path(f"{p}_{k}_{level}"))


def get_args(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    g = p.add_argument_group("input data")
    g.add_argument("--input", required=True, help="JSON-lines file, or a glob when --partitions > 1")
    g.add_argument("--json-keys", nargs="+", default=["text"])
    g.add_argument("--split-sentences", action="store_true")
    g.add_argument("--plain-text", action="store_true", help="input lines are sentences of text, not JSON records")
    g.add_argument("--keep-newlines", action="store_true")
    g = p.add_argument_group("tokenizer")
    g.add_argument("--tokenizer-type", required=True)
    g.add_argument("--tokenizer-model", default=None)
    g.add_argument("--vocab-file", default=None)
    g.add_argument("--merge-file", default=None)
    g.add_argument("--vocab-size", type=int, default=None)
    g.add_argument("--vocab-extra-ids", type=int, default=0)
    g.add_argument("--append-eod", action="store_true")
    g.add_argument("--lang", default="english")
    g = p.add_argument_group("output")
    g.add_argument("--output-prefix", required=True)
    g = p.add_argument_group("runtime")
    g.add_argument("--workers", type=int, default=1)
    g.add_argument("--partitions", type=int, default=1)
    g.add_argument("--log-interval", type=int, default=1000)
    g.add_argument("--keep-sequential-samples", action="store_true")
    a = p.parse_args(argv)
    a.rank, a.make_vocab_size_divisible_by, a.tensor_model_parallel_size, a.padded_vocab_size = 0, 128, 1, None
    return a


def main(argv=None):
    args = get_args(argv)
    if args.partitions == 1:
        process_file(args, args.input, args.output_prefix)
        return
    files = sorted(glob.glob(args.input))
    if len(files) == 1:                              # cut one file into line-interleaved partitions
        stem = args.output_prefix
        outs = [open(f"{stem}_part{i}.jsonl", "w", encoding="utf-8") for i in range(args.partitions)]
        with open(files[0], "r", encoding="utf-8") as f:
            if args.keep_sequential_samples:
                lines = f.readlines()
                per = (len(lines) + args.partitions - 1) // args.partitions
                for i, o in enumerate(outs):
                    o.writelines(lines[i * per:(i + 1) * per])
            else:
                for i, line in enumerate(f):
                    outs[i % args.partitions].write(line)
        for o in outs:
            o.close()
        files = [f"{stem}_part{i}.jsonl" for i in range(args.partitions)]
    parts = []
    for i, fpath in enumerate(files):
        part = f"{args.output_prefix}_{i}"
        process_file(args, fpath, part)
        parts.append(part)
    merge_partitions(args, parts, args.output_prefix)


if __name__ == "__main__":
    main()
