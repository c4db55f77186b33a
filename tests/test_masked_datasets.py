"""BERT / T5 masked datasets over a small sentence-level indexed dataset."""
import numpy as np

from megatron_lm_b200.data.indexed_dataset import IndexedDataset, IndexedDatasetBuilder, get_bin_path, get_idx_path
from megatron_lm_b200.data.masked_dataset import (BERTMaskedWordPieceDataset, MaskedWordPieceDatasetConfig,
                                                  T5MaskedWordPieceDataset)


class _Tok:
    cls, sep, mask, pad, vocab_size = 1, 2, 3, 0, 200
    bos, eos = 1, 2
    additional_special_tokens_ids = list(range(190, 200))


def _dataset(tmp_path):
    prefix = str(tmp_path / "sents")
    b = IndexedDatasetBuilder(get_bin_path(prefix), dtype=np.int32)
    rng = np.random.RandomState(0)
    for _ in range(40):                         # documents of 3-6 sentences
        for _ in range(rng.randint(3, 7)):
            b.add_item(rng.randint(10, 180, size=rng.randint(4, 12)).tolist())
        b.end_document()
    b.finalize(get_idx_path(prefix))
    return IndexedDataset(prefix)


def test_bert_dataset(tmp_path):
    ds = _dataset(tmp_path)
    cfg = MaskedWordPieceDatasetConfig(sequence_length=48, tokenizer=_Tok())
    b = BERTMaskedWordPieceDataset(ds, np.arange(len(ds.document_indices) - 1), 64, "train", cfg)
    assert len(b) >= 64
    s = b[5]
    n = int(s["padding_mask"].sum())
    assert s["text"][0] == 1 and (s["text"][:n] == 2).sum() == 2 and s["text"][n:].sum() == 0
    assert s["loss_mask"].sum() >= 1 and (s["labels"][s["loss_mask"] == 1] >= 10).all()
    assert set(np.unique(s["types"][:n])) <= {0, 1}
    assert (b[5]["text"] == s["text"]).all()           # deterministic per index


def test_t5_dataset(tmp_path):
    ds = _dataset(tmp_path)
    cfg = MaskedWordPieceDatasetConfig(sequence_length=48, sequence_length_decoder=24, tokenizer=_Tok())
    t = T5MaskedWordPieceDataset(ds, np.arange(len(ds.document_indices) - 1), 32, "train", cfg)
    s = t[3]
    sent_in_enc = [x for x in s["text_enc"] if x >= 190]
    assert sent_in_enc and s["text_dec"][0] == 1 and s["text_dec"][1] == sent_in_enc[0]
    assert (s["labels"][s["loss_mask"] == 1] != -1).all()
