"""BERT and T5: padding does not leak, decoder is causal, losses train."""
import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.bert import BertModel
from megatron_lm_b200.models.t5 import T5Model


def _cfg(**kw):
    return TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                             hidden_dropout=0.0, attention_dropout=0.0, **kw)


def test_bert_padding_and_heads():
    torch.manual_seed(0)
    m = BertModel(_cfg(), num_tokentypes=2, vocab_size=64, max_sequence_length=16,
                  share_embeddings_and_output_weights=True).eval()
    ids = torch.randint(0, 64, (2, 12)); mask = torch.ones(2, 12); mask[:, 8:] = 0
    tt = torch.zeros(2, 12, dtype=torch.long)
    with torch.no_grad():
        a, nsp = m(ids, mask, tt)
        ids2 = ids.clone(); ids2[:, 8:] = 3                      # change only padded tokens
        b, _ = m(ids2, mask, tt)
    assert a.shape == (2, 12, 64) and nsp.shape == (2, 2)
    assert torch.allclose(a[:, :8], b[:, :8], atol=1e-5)
    m.train()
    loss, nsp = m(ids, mask, tt, lm_labels=ids)
    (loss.mean() + nsp.float().sum() * 0).backward()
    w = m.embedding.word_embeddings.weight
    g = w.grad if w.grad is not None else w.main_grad
    assert torch.isfinite(g).all() and g.abs().sum() > 0


def test_t5_causal_decoder_and_cross_mask():
    torch.manual_seed(0)
    m = T5Model(_cfg(), vocab_size=64, max_sequence_length=16).eval()
    enc = torch.randint(0, 64, (2, 10)); dec = torch.randint(0, 64, (2, 6))
    em = torch.ones(2, 10); em[:, 7:] = 0
    enc_mask = em.unsqueeze(1) * em.unsqueeze(2)
    x_mask = torch.ones(2, 6, 1) * em.unsqueeze(1)
    with torch.no_grad():
        a = m(enc, dec, enc_mask, None, x_mask)
        dec2 = dec.clone(); dec2[:, 4:] = 5
        b = m(enc, dec2, enc_mask, None, x_mask)
        enc2 = enc.clone(); enc2[:, 7:] = 9
        c = m(enc2, dec, enc_mask, None, x_mask)
    assert a.shape == (2, 6, 64)
    assert torch.allclose(a[:, :4], b[:, :4], atol=1e-5)          # decoder is causal
    assert torch.allclose(a, c, atol=1e-5)                        # padded encoder tokens are invisible
    m.train()
    loss = m(enc, dec, enc_mask, None, x_mask, lm_labels=dec).mean()
    loss.backward()


def test_bert_embedding_tool(tmp_path):
    """One vector per line, independent of batching and of the other texts in a batch, written in input order."""
    import numpy as np
    from megatron_lm_b200.data import bert_embedding as be
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("\n".join(["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + [f"w{i}" for i in range(40)]) + "\n")
    texts = ["w1 w2 w3", "w4", "w5 w6 w7 w8 w9 w10 w11", "w2 w2"]
    (tmp_path / "in.txt").write_text("\n".join(texts) + "\n")
    flags = ["--num-layers", "2", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "16",
             "--max-position-embeddings", "16", "--tokenizer-type", "BertWordPieceLowerCase", "--vocab-file", str(vocab),
             "--use-cpu-initialization", "--attention-dropout", "0", "--hidden-dropout", "0", "--train-iters", "1",
             "--lr", "1e-3", "--input", str(tmp_path / "in.txt"), "--output", str(tmp_path / "emb.npy"),
             "--output-bert-embeddings", "--seed", "3"]
    torch.manual_seed(0)
    emb = be.main(flags + ["--embed-batch-size", "2"])
    assert emb.shape == (4, 32) and np.isfinite(emb).all() and np.array_equal(np.load(tmp_path / "emb.npy"), emb)
    torch.manual_seed(0)
    one = be.main(flags + ["--embed-batch-size", "1"])
    assert np.allclose(emb, one, atol=1e-5)
    assert not np.allclose(emb[0], emb[1], atol=1e-3)
    import pytest
    with pytest.raises(SystemExit):
        be.main([f for f in flags if f != "--output-bert-embeddings"])
    ds = be.BertEmbeddingDataset(["w1 " * 40], __import__("megatron_lm_b200.data.tokenizer", fromlist=["x"]).build_tokenizer(
        __import__("types").SimpleNamespace(tokenizer_type="BertWordPieceLowerCase", vocab_file=str(vocab), rank=0,
                                            make_vocab_size_divisible_by=1, tensor_model_parallel_size=1,
                                            vocab_extra_ids=0, padded_vocab_size=None)), 16)
    item = ds[0]
    assert item["length"] == 16 and item["text"][0] == 2 and item["text"][-1] == 3
