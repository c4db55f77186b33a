"""Concatenate every indexed dataset (``.bin`` + ``.idx`` pair) of a directory into one.

``python -m megatron_lm_b200.data.merge_datasets --input dir --output-prefix merged``
(reference: tools/merge_datasets.py).
"""
from __future__ import annotations

import argparse
import os

from .indexed_dataset import IndexedDataset, IndexedDatasetBuilder, get_bin_path, get_idx_path


def merge(input_dir: str, output_prefix: str, multimodal: bool = False) -> int:
    prefixes = set()
    for name in os.listdir(input_dir):
        stem, ext = os.path.splitext(name)
        if ext in (".bin", ".idx"):
            other = stem + (".idx" if ext == ".bin" else ".bin")
            if not os.path.isfile(os.path.join(input_dir, other)):
                raise FileNotFoundError(f"{name} has no matching {other}")
            prefixes.add(os.path.join(input_dir, stem))
    builder = None
    for prefix in sorted(prefixes):
        if builder is None:
            ds = IndexedDataset(prefix, multimodal=multimodal)
            builder = IndexedDatasetBuilder(get_bin_path(output_prefix), dtype=ds.index.dtype, multimodal=multimodal)
            del ds
        builder.add_index(prefix)
    if builder is None:
        raise FileNotFoundError(f"no indexed datasets in {input_dir}")
    builder.finalize(get_idx_path(output_prefix))
    return len(prefixes)


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--input", required=True)
    p.add_argument("--output-prefix", required=True)
    p.add_argument("--multimodal", action="store_true")
    a = p.parse_args(argv)
    n = merge(a.input, a.output_prefix, a.multimodal)
    print(f"merged {n} datasets into {a.output_prefix}")


if __name__ == "__main__":
    main()
