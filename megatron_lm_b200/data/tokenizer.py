"""Tokenizer front-ends selected by ``--tokenizer-type`` (reference:
megatron/training/tokenizer/tokenizer.py: build_tokenizer :21, vocab padding :115, HF :131,
BertWordPiece :193, GPT2BPE :329, SentencePiece :363, Llama2 :573, TikToken :662, Null :801).
Each exposes ``vocab_size``, ``tokenize``, ``detokenize`` and the special ids training needs
(``eod``, ``pad``, ``bos``, ``eos``, ``cls``, ``sep``, ``mask`` where defined)."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional


def vocab_size_with_padding(orig_vocab_size: int, make_vocab_size_divisible_by: int = 128,
                            tensor_model_parallel_size: int = 1) -> int:
    """Pad the vocabulary so that it splits evenly over TP ranks in multiples of the alignment."""
    multiple = make_vocab_size_divisible_by * tensor_model_parallel_size
    return ((orig_vocab_size + multiple - 1) // multiple) * multiple


class MegatronTokenizer:
    def __init__(self, name: str):
        self.name = name

    @property
    def vocab_size(self) -> int:
        raise NotImplementedError

    def tokenize(self, text: str) -> List[int]:
        raise NotImplementedError

    def detokenize(self, ids: List[int]) -> str:
        raise NotImplementedError

    @property
    def eod(self) -> int:
        raise NotImplementedError

    pad = None
    bos = None
    eos = None
    cls = None
    sep = None
    mask = None


class NullTokenizer(MegatronTokenizer):
    """Whitespace-separated integers; the id ``vocab_size`` itself is EOD."""

    def __init__(self, vocab_size: int):
        super().__init__("NullTokenizer")
        self._vocab_size_without_eod = int(vocab_size)
        self._eod = int(vocab_size)

    def tokenize(self, text):
        return [int(x) for x in text.split(" ")]

    def detokenize(self, ids):
        return " ".join(str(i) for i in ids)

    @property
    def vocab_size(self):
        return self._vocab_size_without_eod + 1

    @property
    def eod(self):
        return self._eod

    @property
    def cls(self):
        return -1

    @property
    def sep(self):
        return -1

    @property
    def mask(self):
        return -1

    @property
    def pad(self):
        return -1


def _bytes_to_unicode() -> Dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, [chr(c) for c in cs]))


class GPT2BPETokenizer(MegatronTokenizer):
    """Byte-level BPE from a ``vocab.json`` + ``merges.txt`` pair."""

    def __init__(self, vocab_file: str, merge_file: str):
        super().__init__("GPT2BPETokenizer")
        import regex as re
        with open(vocab_file, encoding="utf-8") as f:
            self.encoder = json.load(f)
        self.decoder = {v: k for k, v in self.encoder.items()}
        with open(merge_file, encoding="utf-8") as f:
            merges = [tuple(l.split()) for l in f.read().split("\n")[1:] if l and not l.startswith("#")]
        self.bpe_ranks = {m: i for i, m in enumerate(merges) if len(m) == 2}
        self.byte_encoder = _bytes_to_unicode()
        self.byte_decoder = {v: k for k, v in self.byte_encoder.items()}
        self.pat = re.compile(r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""")
        self.cache: Dict[str, str] = {}
        self.eod_id = self.encoder["<|endoftext|>"]

    def _bpe(self, token: str) -> str:
        if token in self.cache:
            return self.cache[token]
        word = tuple(token)
        while len(word) > 1:
            pairs = set(zip(word[:-1], word[1:]))
            best = min(pairs, key=lambda p: self.bpe_ranks.get(p, float("inf")))
            if best not in self.bpe_ranks:
                break
            a, b = best
            new, i = [], 0
            while i < len(word):
                if i < len(word) - 1 and word[i] == a and word[i + 1] == b:
                    new.append(a + b)
                    i += 2
                else:
                    new.append(word[i])
                    i += 1
            word = tuple(new)
        out = " ".join(word)
        self.cache[token] = out
        return out

    def tokenize(self, text):
        ids = []
        for tok in self.pat.findall(text):
            tok = "".join(self.byte_encoder[b] for b in tok.encode("utf-8"))
            ids.extend(self.encoder[t] for t in self._bpe(tok).split(" "))
        return ids

    def detokenize(self, ids):
        text = "".join(self.decoder[i] for i in ids)
        return bytearray([self.byte_decoder[c] for c in text]).decode("utf-8", errors="replace")

    @property
    def vocab_size(self):
        return len(self.encoder)

    @property
    def vocab(self):
        return self.encoder

    @property
    def inv_vocab(self):
        return self.decoder

    @property
    def eod(self):
        return self.eod_id


class SentencePieceTokenizer(MegatronTokenizer):
    def __init__(self, model_file: str, vocab_extra_ids: int = 0, legacy: bool = True):
        super().__init__("SentencePieceTokenizer")
        import sentencepiece
        self.sp = sentencepiece.SentencePieceProcessor(model_file=model_file)
        self._vocab = {self.sp.id_to_piece(i): i for i in range(len(self.sp))}
        self._inv = {i: p for p, i in self._vocab.items()}
        self._special: Dict[str, int] = {}

        def add(tok):
            if tok not in self._vocab:
                i = len(self._vocab)
                self._vocab[tok] = i
                self._inv[i] = tok
            self._special[tok] = self._vocab[tok]
            return self._vocab[tok]
        if legacy:
            self._cls, self._sep, self._eod_, self._mask = add("<CLS>"), add("<SEP>"), add("<EOD>"), add("<MASK>")
        self._pad = self.sp.pad_id() if self.sp.pad_id() >= 0 else (add("<PAD>") if legacy else -1)
        self._bos = self.sp.bos_id() if self.sp.bos_id() >= 0 else (add("<BOS>") if legacy else -1)
        self._eos = self.sp.eos_id() if self.sp.eos_id() >= 0 else (add("<EOS>") if legacy else -1)
        if not legacy:
            self._eod_ = self._eos
        for i in range(vocab_extra_ids):
            add(f"<extra_id_{i}>")

    def tokenize(self, text):
        return self.sp.encode_as_ids(text)

    def detokenize(self, ids):
        n = len(self.sp)
        return self.sp.decode_ids([i for i in ids if i < n])

    @property
    def vocab_size(self):
        return len(self._vocab)

    @property
    def eod(self):
        return self._eod_

    @property
    def pad(self):
        return self._pad

    @property
    def bos(self):
        return self._bos

    @property
    def eos(self):
        return self._eos


class Llama2Tokenizer(SentencePieceTokenizer):
    def __init__(self, model_file: str):
        super().__init__(model_file, 0, legacy=False)
        self.name = "Llama2Tokenizer"

    def tokenize(self, text, bos: bool = True, eos: bool = False):
        ids = self.sp.encode(text)
        return ([self._bos] if bos else []) + ids + ([self._eos] if eos else [])


class HuggingFaceTokenizer(MegatronTokenizer):
    def __init__(self, pretrained_model_name_or_path: str, **kw):
        super().__init__("HuggingFaceTokenizer")
        import transformers
        self._tok = transformers.AutoTokenizer.from_pretrained(pretrained_model_name_or_path, **kw)

    def tokenize(self, text, **kw):
        return self._tok(text, **kw).input_ids

    def detokenize(self, ids, **kw):
        return self._tok.decode(ids, **kw)

    @property
    def vocab_size(self):
        return len(self._tok)

    @property
    def eod(self):
        return self._tok.eos_token_id

    @property
    def pad(self):
        return self._tok.pad_token_id

    @property
    def bos(self):
        return self._tok.bos_token_id

    @property
    def eos(self):
        return self._tok.eos_token_id


class TikTokenizer(MegatronTokenizer):
    """tiktoken BPE from a json vocabulary of {rank, token_bytes(base64), token_str} entries."""

    def __init__(self, path: str, pattern: str = "v1", vocab_size: Optional[int] = None, num_special_tokens: int = 1000,
                 special_tokens: Optional[List[str]] = None):
        super().__init__("TikTokenizer")
        import base64
        import tiktoken
        pats = {"v1": r"""[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+|[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+""",
                "v2": r"[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"}
        specials = list(special_tokens or ["<unk>", "<s>", "</s>"])
        specials += [f"<SPECIAL_{i}>" for i in range(len(specials), num_special_tokens)]
        with open(path) as f:
            entries = json.load(f)
        ranks = {base64.b64decode(e["token_bytes"]): e["rank"] for e in entries}
        if vocab_size is not None:
            ranks = {k: v for k, v in ranks.items() if v < vocab_size - num_special_tokens}
        self.num_special = num_special_tokens
        self._specials = specials
        self._model = tiktoken.Encoding(name=os.path.basename(path), pat_str=pats.get(pattern, pattern),
                                        mergeable_ranks=ranks, special_tokens={})
        self._n = len(ranks) + num_special_tokens
        self._unk, self._bos, self._eos = (specials.index(t) for t in ("<unk>", "<s>", "</s>"))

    def tokenize(self, text, bos: bool = False, eos: bool = False):
        ids = [t + self.num_special for t in self._model.encode_ordinary(text)]
        return ([self._bos] if bos else []) + ids + ([self._eos] if eos else [])

    def detokenize(self, ids):
        return self._model.decode([t - self.num_special for t in ids if t >= self.num_special])

    @property
    def vocab_size(self):
        return self._n

    @property
    def eod(self):
        return self._eos

    @property
    def bos(self):
        return self._bos

    @property
    def eos(self):
        return self._eos

    @property
    def pad(self):
        return self._unk


class BertWordPieceTokenizer(MegatronTokenizer):
    """Greedy longest-match WordPiece over a one-token-per-line vocabulary file."""

    def __init__(self, vocab_file: str, lower_case: bool = True, vocab_extra_ids: int = 0):
        super().__init__("BertWordPieceTokenizer")
        with open(vocab_file, encoding="utf-8") as f:
            toks = [l.rstrip("\n") for l in f]
        self.vocab_ = {t: i for i, t in enumerate(toks)}
        for i in range(vocab_extra_ids):
            self.vocab_.setdefault(f"<extra_id_{i}>", len(self.vocab_))
        for t in ("[BOS]", "[EOS]"):
            self.vocab_.setdefault(t, len(self.vocab_))
        self.inv = {i: t for t, i in self.vocab_.items()}
        self.lower = lower_case

    def _basic(self, text: str) -> List[str]:
        import unicodedata
        if self.lower:
            text = unicodedata.normalize("NFD", text.lower())
            text = "".join(c for c in text if unicodedata.category(c) != "Mn")
        out, cur = [], ""
        for c in text:
            if c.isspace():
                if cur:
                    out.append(cur)
                    cur = ""
            elif unicodedata.category(c).startswith("P") or (33 <= ord(c) <= 47) or (58 <= ord(c) <= 64) or \
                    (91 <= ord(c) <= 96) or (123 <= ord(c) <= 126):
                if cur:
                    out.append(cur)
                    cur = ""
                out.append(c)
            else:
                cur += c
        if cur:
            out.append(cur)
        return out

    def tokenize(self, text):
        ids = []
        unk = self.vocab_.get("[UNK]", 0)
        for w in self._basic(text):
            start, pieces, bad = 0, [], False
            while start < len(w):
                end, cur = len(w), None
                while start < end:
                    sub = ("##" if start > 0 else "") + w[start:end]
                    if sub in self.vocab_:
                        cur = sub
                        break
                    end -= 1
                if cur is None:
                    bad = True
                    break
                pieces.append(self.vocab_[cur])
                start = end
            ids.extend([unk] if bad else pieces)
        return ids

    def detokenize(self, ids):
        toks = [self.inv[i] for i in ids]
        out = ""
        for t in toks:
            out += t[2:] if t.startswith("##") else ((" " if out else "") + t)
        return out

    @property
    def vocab_size(self):
        return len(self.vocab_)

    @property
    def vocab(self):
        return self.vocab_

    @property
    def cls(self):
        return self.vocab_["[CLS]"]

    @property
    def sep(self):
        return self.vocab_["[SEP]"]

    @property
    def pad(self):
        return self.vocab_["[PAD]"]

    @property
    def mask(self):
        return self.vocab_["[MASK]"]

    @property
    def eod(self):
        return self.vocab_["[EOS]"]

    @property
    def bos(self):
        return self.vocab_["[BOS]"]

    @property
    def eos(self):
        return self.vocab_["[EOS]"]

    @property
    def additional_special_tokens_ids(self):
        """The sentinel ids ``<extra_id_i>`` added by ``vocab_extra_ids`` (T5 span corruption)."""
        return [i for t, i in self.vocab_.items() if t.startswith("<extra_id_")]

    @property
    def eos(self):
        return self.vocab_["[EOS]"]


def build_tokenizer(args):
    """Instantiate the tokenizer named by ``args.tokenizer_type`` and set ``args.padded_vocab_size``."""
    t = args.tokenizer_type
    if t == "NullTokenizer":
        tok = NullTokenizer(args.vocab_size)
    elif t == "GPT2BPETokenizer":
        tok = GPT2BPETokenizer(args.vocab_file, args.merge_file)
    elif t in ("BertWordPieceLowerCase", "BertWordPieceCase"):
        tok = BertWordPieceTokenizer(args.vocab_file, t.endswith("LowerCase"), getattr(args, "vocab_extra_ids", 0))
    elif t in ("SentencePieceTokenizer", "GPTSentencePieceTokenizer"):
        tok = SentencePieceTokenizer(args.tokenizer_model, getattr(args, "vocab_extra_ids", 0),
                                     legacy=(t == "SentencePieceTokenizer"))
    elif t == "Llama2Tokenizer":
        tok = Llama2Tokenizer(args.tokenizer_model)
    elif t == "HuggingFaceTokenizer":
        tok = HuggingFaceTokenizer(args.tokenizer_model)
    elif t == "TikTokenizer":
        tok = TikTokenizer(args.tokenizer_model, getattr(args, "tiktoken_pattern", "v1"), getattr(args, "vocab_size", None),
                           getattr(args, "tiktoken_num_special_tokens", 1000),
                           getattr(args, "tiktoken_special_tokens", None))
    else:
        raise NotImplementedError(f"tokenizer {t} is not implemented")
    if getattr(args, "padded_vocab_size", None) is None:
        args.padded_vocab_size = vocab_size_with_padding(tok.vocab_size,
                                                         getattr(args, "make_vocab_size_divisible_by", 128),
                                                         getattr(args, "tensor_model_parallel_size", 1))
    return tok
