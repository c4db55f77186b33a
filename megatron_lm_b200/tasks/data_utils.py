"""Sample construction for sentence / sentence-pair tasks: [CLS] a [SEP] (b [SEP]) with token types and padding.

Reference: tasks/data_utils.py:9-105 (``clean_text``, ``build_sample``,
``build_tokens_types_paddings_from_text`` / ``_from_ids``)."""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


def clean_text(text: str) -> str:
    """Newlines to spaces, runs of white space to one space, `` . `` glued back to the sentence."""
    text = text.replace("\n", " ")
    text = re.sub(r"\s+", " ", text)
    for _ in range(3):
        text = text.replace(" . ", ". ")
    return text


def build_sample(ids: Sequence[int], types: Sequence[int], paddings: Sequence[int], label: int, unique_id: int) -> Dict:
    return {"text": np.array(ids, dtype=np.int64), "types": np.array(types, dtype=np.int64),
            "padding_mask": np.array(paddings, dtype=np.int64), "label": int(label), "uid": int(unique_id)}


def build_tokens_types_paddings_from_ids(a_ids: Sequence[int], b_ids: Optional[Sequence[int]], max_seq_length: int,
                                         cls_id: int, sep_id: int, pad_id: int) -> Tuple[List[int], List[int], List[int]]:
    """[CLS] A [SEP] B [SEP], token types 0 for the A part and 1 for the B part, truncated to ``max_seq_length``
    (the final [SEP] survives a truncation), then padded; the padding mask is 1 on real tokens."""
    ids, types = [cls_id], [0]
    ids.extend(a_ids)
    types.extend([0] * len(a_ids))
    ids.append(sep_id)
    types.append(0)
    if b_ids is not None:
        ids.extend(b_ids)
        types.extend([1] * len(b_ids))
    trimmed = False
    if len(ids) >= max_seq_length:
        ids, types, trimmed = ids[:max_seq_length - 1], types[:max_seq_length - 1], True
    if b_ids is not None or trimmed:
        ids.append(sep_id)
        types.append(1 if b_ids is not None else 0)
    paddings = [1] * len(ids)
    n_pad = max_seq_length - len(ids)
    if n_pad > 0:
        ids.extend([pad_id] * n_pad)
        types.extend([pad_id] * n_pad)
        paddings.extend([0] * n_pad)
    return ids, types, paddings


def build_tokens_types_paddings_from_text(text_a: str, text_b: Optional[str], tokenizer, max_seq_length: int):
    a = tokenizer.tokenize(text_a)
    b = tokenizer.tokenize(text_b) if text_b is not None else None
    return build_tokens_types_paddings_from_ids(a, b, max_seq_length, tokenizer.cls, tokenizer.sep, tokenizer.pad)
