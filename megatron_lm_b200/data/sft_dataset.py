"""Supervised fine-tuning dataset: chat conversations packed to a fixed length, loss on assistant turns only.

Reference: megatron/training/datasets/sft_dataset.py (``SFTLowLevelDataset`` :17, ``SFTDataset`` :46):
conversations are lists of {"role", "content"} messages; tokens of non-assistant turns and padding get
loss mask 0; one conversation per sample, truncated or padded to ``sequence_length + 1``.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

import numpy as np
import torch

IGNORE_INDEX = -100


class SFTLowLevelDataset:
    """JSON-lines file; each line either a list of messages or {"messages" | "conversations": [...]}"""

    def __init__(self, path: str):
        self.rows = []
        with open(path, "r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                obj = json.loads(line)
                if isinstance(obj, dict):
                    obj = obj.get("messages", obj.get("conversations"))
                self.rows.append(obj)

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]


def default_chat_template(role: str, content: str) -> str:
    return f"<|{role}|>\n{content}\n"


def identity_template(role: str, content: str) -> str:
    """The turn's text as it is (pre-formatted or pre-tokenised conversations)."""
    return content


TEMPLATES = {"identity": identity_template}


class SFTDataset(torch.utils.data.Dataset):
    def __init__(self, dataset, tokenizer, sequence_length: int, num_samples: Optional[int] = None,
                 template=default_chat_template, pad_id: Optional[int] = None, seed: int = 1234):
        self.ds = SFTLowLevelDataset(dataset) if isinstance(dataset, str) else dataset
        self.tok, self.seq, self.template = tokenizer, sequence_length, template
        if pad_id is None:
            try:
                pad_id = tokenizer.pad
            except (AttributeError, NotImplementedError):
                pad_id = None
        self.pad = tokenizer.eod if pad_id is None else pad_id
        n = num_samples or len(self.ds)
        rng = np.random.RandomState(seed)
        order = []
        while len(order) < n:
            order.extend(rng.permutation(len(self.ds)).tolist())
        self.order = order[:n]

    def __len__(self):
        return len(self.order)

    def tokenize_conversation(self, messages: List[Dict[str, str]]):
        tokens, targets = [], []
        for m in messages:
            role = m.get("role", m.get("from"))
            ids = self.tok.tokenize(self.template(role, m.get("content", m.get("value", ""))))
            tokens.extend(ids)
            targets.extend(ids if role in ("assistant", "gpt") else [IGNORE_INDEX] * len(ids))
        tokens.append(self.tok.eod)
        targets.append(self.tok.eod if messages and messages[-1].get("role", messages[-1].get("from")) in
                       ("assistant", "gpt") else IGNORE_INDEX)
        return tokens, targets

    def __getitem__(self, i):
        tokens, targets = self.tokenize_conversation(self.ds[self.order[i]])
        L = self.seq + 1
        tokens, targets = tokens[:L], targets[:L]
        pad = L - len(tokens)
        tokens = tokens + [self.pad] * pad
        targets = targets + [IGNORE_INDEX] * pad
        t = torch.tensor(tokens, dtype=torch.int64)
        y = torch.tensor(targets, dtype=torch.int64)
        labels = y[1:].clone()
        loss_mask = (labels != IGNORE_INDEX).float()
        labels[labels == IGNORE_INDEX] = self.pad
        return {"tokens": t[:-1].contiguous(), "labels": labels, "loss_mask": loss_mask,
                "position_ids": torch.arange(self.seq, dtype=torch.int64)}
