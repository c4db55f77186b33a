"""Zero-shot language-model evaluation: perplexity over a long text (WikiText-103 style) and last-word
accuracy (LAMBADA style).

Reference: tasks/zeroshot_gpt/evaluate.py (``forward_step`` :68, ``evaluate`` :113,
``evaluate_and_print_results`` :147) and datasets.py (``_LMDataset`` :35 overlapping windows,
``_LambadaDataset`` :80), detokenizer.py (WikiText clean-up rules).
"""
from __future__ import annotations

import json
import math
import re
from typing import Dict, List, Optional

import torch


def wikitext_detokenizer(s: str) -> str:
    s = s.replace("s '", "s'")
    s = re.sub(r"/' [0-9]/", r"/'[0-9]/", s)
    s = s.replace(" @-@ ", "-").replace(" @,@ ", ",").replace(" @.@ ", ".")
    s = s.replace(" : ", ": ").replace(" ; ", "; ").replace(" . ", ". ").replace(" ! ", "! ").replace(" ? ", "? ")
    s = s.replace(" , ", ", ")
    s = re.sub(r"\(\s*([^\)]*?)\s*\)", r"(\1)", s)
    s = re.sub(r"\[\s*([^\]]*?)\s*\]", r"[\1]", s)
    s = re.sub(r"{\s*([^}]*?)\s*}", r"{\1}", s)
    s = re.sub(r"\"\s*([^\"]*?)\s*\"", r'"\1"', s)
    s = re.sub(r"'\s*([^']*?)\s*'", r"'\1'", s)
    s = s.replace("= = = =", "====").replace("= = =", "===").replace("= =", "==")
    s = s.replace(" " + chr(176) + " ", chr(176)).replace(" \n", "\n").replace("\n ", "\n")
    s = s.replace(" N ", " 1 ").replace(" 's", "'s")
    return s


class LMDataset(torch.utils.data.Dataset):
    """Overlapping windows over one token stream; only the tokens not scored by the previous window count."""

    def __init__(self, tokens: List[int], seq_len: int, pad_idx: int, num_original_tokens: int,
                 num_tokenized_tokens: int, overlapping_eval: Optional[int] = None):
        self.tokens, self.seq_len, self.pad_idx = tokens, seq_len, pad_idx
        self.overlap = max(1, overlapping_eval or seq_len)
        self.num_original_tokens, self.num_tokenized_tokens = num_original_tokens, num_tokenized_tokens
        targets = max(len(tokens) - 1, 0)
        self.total_sequences = max(math.ceil(max(targets - seq_len, 0) / self.overlap) + 1, 1)

    def __len__(self):
        return self.total_sequences

    def __getitem__(self, idx):
        start = idx * self.overlap
        toks = self.tokens[start:start + self.seq_len + 1]
        n = len(toks)
        mask = [1] * n + [0] * (self.seq_len + 1 - n)
        toks = toks + [self.pad_idx] * (self.seq_len + 1 - n)
        mask = mask[1:]
        if self.overlap != self.seq_len and idx != 0:
            mask[:-self.overlap] = [0] * (len(mask) - self.overlap)
        return {"text": torch.tensor(toks), "pad_mask": torch.tensor(mask)}


class LambadaDataset(torch.utils.data.Dataset):
    def __init__(self, path: str, pad_idx: int, tokenizer, seq_len: int, strict: bool = False):
        self.seq_len, self.pad_idx, self.tok, self.strict = seq_len, pad_idx, tokenizer, strict
        self.tokens, self.labels = [], []
        with open(path) as f:
            for line in f:
                text = json.loads(line)["text"]
                t, l = self._split(text)
                self.tokens.append(t)
                self.labels.append(l)

    def _split(self, text):
        if not self.strict:
            t = self.tok.tokenize(text)
            return t[:-1], [t[-1]]
        last = text.split()[-1]
        start = text.rfind(last)
        return self.tok.tokenize(text[:start].strip()), self.tok.tokenize(" " + last)

    def __len__(self):
        return len(self.tokens)

    def __getitem__(self, i):
        t, l = self.tokens[i], self.labels[i]
        toks = t + l
        mask = [0] * len(t) + [1] * len(l)
        pad = self.seq_len + 1 - len(toks)
        return {"text": torch.tensor(toks + [self.pad_idx] * pad), "pad_mask": torch.tensor((mask + [0] * pad)[1:])}


@torch.no_grad()
def evaluate(model, loader, task: str = "WIKITEXT103") -> float:
    """Sum of masked token losses (perplexity tasks) or count of fully correct continuations (LAMBADA)."""
    model.eval()
    total = 0.0
    dev = next(model.parameters()).device
    for batch in loader:
        toks = batch["text"].to(dev)
        mask = batch["pad_mask"].to(dev).float()
        inp, labels = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()
        if task.upper().startswith("LAMBADA"):
            logits = model(inp)
            correct = (logits.argmax(-1) == labels).float()
            correct = torch.where(mask > 0, correct, torch.ones_like(correct))
            total += float(correct.prod(-1).sum())
        else:
            losses = model(inp, labels=labels).float()
            total += float((losses * mask).sum())
    return total


def results(task: str, total: float, dataset) -> Dict[str, float]:
    if task.upper().startswith("LAMBADA"):
        n = len(dataset)
        return {"number correct": total, "total examples": n, "avg accuracy": total / max(n, 1)}
    val = total / max(dataset.num_tokenized_tokens - 1, 1)
    ratio = (dataset.num_tokenized_tokens - 1) / max(dataset.num_original_tokens - 1, 1)
    return {"avg loss": val, "ppl": math.exp(min(20, val)), "adjusted ppl": math.exp(min(20, val * ratio)),
            "token ratio": ratio}
