"""Evidence embedding store, exact inner-product search, the evidence dataset and the indexing program (reference:
megatron/legacy/data/realm_index.py, orqa_wiki_dataset.py, megatron/legacy/indexer.py)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from megatron_lm_b200.data.retrieval_index import (
    BlockEmbeddingStore, IndexBuilder, MIPSIndex, OpenRetrievalEvidenceDataset, retrieval_topk_accuracy)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _evidence(tmp_path, n=23):
    path = tmp_path / "evidence.tsv"
    rng = np.random.RandomState(3)
    lines = ["id\ttext\ttitle"]
    for i in range(n):
        text = " ".join(f"w{int(t)}" for t in rng.randint(0, 60, size=rng.randint(5, 40)))
        lines.append(f"{100 + i}\t{text}\tw{i % 7} w{i % 5}")
    path.write_text("\n".join(lines) + "\n")
    vocab = tmp_path / "vocab.txt"
    vocab.write_text("\n".join(["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + [f"w{i}" for i in range(60)]) + "\n")
    return str(path), str(vocab)


def test_store_shards_merge_and_reload(tmp_path):
    path = str(tmp_path / "embeds.pt")
    a, b = BlockEmbeddingStore(path, rank=0), BlockEmbeddingStore(path, rank=1)
    a.add_block_data([0, 2, 4], torch.arange(12.0).view(3, 4))
    b.add_block_data(torch.tensor([1, 3]), torch.arange(12.0, 20.0).view(2, 4))
    with pytest.raises(ValueError, match="twice"):
        a.add_block_data([2], torch.zeros(1, 4))
    b.save_shard()
    a.save_shard()
    assert a.merge_shards_and_save() == 2 and len(a) == 5
    assert not os.path.exists(a.temp_dir)
    again = BlockEmbeddingStore(path, load_from_path=True)
    st = again.state()
    assert st["row_ids"].tolist() == [0, 1, 2, 3, 4] and st["embeds"].dtype == torch.float16
    torch.testing.assert_close(st["embeds"][1].float(), torch.arange(12.0, 16.0))


def test_mips_search_is_exact_across_blocks():
    torch.manual_seed(0)
    embeds, ids = torch.randn(500, 16), torch.randperm(5000)[:500]
    index = MIPSIndex(16, device="cpu", block_rows=64)
    index.add(ids[:300], embeds[:300])
    index.add(ids[300:], embeds[300:])
    q = torch.randn(7, 16)
    scores, found = index.search_mips_index(q, 10)
    want_s, want_j = (q @ embeds.t()).topk(10, dim=1)
    torch.testing.assert_close(scores, want_s)
    assert torch.equal(found, ids[want_j])
    assert index.search_mips_index(q, 1000)[1].shape == (7, 500)          # k is capped by the index size
    acc = retrieval_topk_accuracy(index, embeds[:50] * 3, [[int(i)] for i in ids[:50]], ks=(1, 5))
    own = (embeds[:50] @ embeds.t()).argmax(dim=1)                        # inner products favour long rows
    assert abs(acc[1] - float((own == torch.arange(50)).float().mean())) < 1e-6 and acc[5] >= acc[1] > 0.5
    with pytest.raises(ValueError, match="wide"):
        index.add(ids[:2], torch.randn(2, 8))


def test_evidence_dataset_and_index_builder(tmp_path):
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.data.tokenizer import BertWordPieceTokenizer
    from megatron_lm_b200.models.bert import BiEncoderModel
    path, vocab = _evidence(tmp_path)
    tk = BertWordPieceTokenizer(vocab, lower_case=True)
    ds = OpenRetrievalEvidenceDataset(path, tk, 24)
    assert len(ds) == 23 and ds.id2text[100][1] == "w0 w0"
    s = ds[3]
    assert s["row_id"] == 103 and s["context"][0] == tk.cls and s["context"].shape == (24,)
    n = int(s["context_pad_mask"].sum())
    assert s["context"][n - 1] == tk.sep and (s["context"][n:] == tk.pad).all()
    assert list(s["context"][1:3]) == tk.tokenize("w3 w3") and s["context"][3] == tk.sep
    assert len(OpenRetrievalEvidenceDataset(path, tk, 24, sample_rate=0.5)) == 11
    torch.manual_seed(1)
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, use_cpu_initialization=True,
                            params_dtype=torch.float32, hidden_dropout=0.0, attention_dropout=0.0)
    model = BiEncoderModel(cfg, 72, 32, projection_dim=8)
    out = str(tmp_path / "index" / "embeds.pt")
    os.makedirs(os.path.dirname(out))
    logs = []
    # two data-parallel builders, run one after the other: the second one to finish merges
    assert IndexBuilder(model, ds, out, batch_size=4, dp_rank=1, dp_size=2).build_and_save_index() == 0
    total = IndexBuilder(model, ds, out, batch_size=4, log_interval=2, dp_rank=0, dp_size=2, log=logs.append).build_and_save_index()
    assert total == 23 and logs and logs[0].startswith("Batch")
    store = BlockEmbeddingStore(out, load_from_path=True)
    assert sorted(store.embed_data) == list(range(100, 123))
    # a stored row is the context tower's embedding of that row
    row = ds[5]
    with torch.no_grad():
        model.eval()
        e = model._embed(model.context_model, torch.as_tensor(row["context"])[None], torch.as_tensor(row["context_pad_mask"])[None],
                         torch.as_tensor(row["context_types"])[None])[0]
    torch.testing.assert_close(store.embed_data[105].float(), e, atol=2e-3, rtol=2e-3)
    index = MIPSIndex(8, store, device="cpu")
    scores, found = index.search_mips_index(e[None], 23)
    assert sorted(found[0].tolist()) == list(range(100, 123))
    all_rows = torch.stack([store.embed_data[i].float() for i in found[0].tolist()])
    torch.testing.assert_close(scores[0], all_rows @ e, atol=1e-3, rtol=1e-3)
    assert retrieval_topk_accuracy(index, e[None], [[105]], ks=(23,))[23] == 1.0


def test_indexing_program_embeds_an_evidence_file(tmp_path):
    path, vocab = _evidence(tmp_path)
    out = str(tmp_path / "embeds.pt")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1", MASTER_PORT="29671")
    cmd = [sys.executable, "-m", "megatron_lm_b200.tasks.build_evidence_index", "--num-layers", "2", "--hidden-size", "32",
           "--num-attention-heads", "4", "--seq-length", "32", "--max-position-embeddings", "64", "--micro-batch-size", "2",
           "--use-cpu-initialization", "--vocab-file", vocab, "--evidence-data-path", path, "--embedding-path", out,
           "--indexer-batch-size", "8", "--indexer-log-interval", "1", "--retriever-seq-length", "24",
           "--biencoder-projection-dim", "16"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "saved 23 embeddings" in r.stdout and "Batch" in r.stdout
    st = torch.load(out, weights_only=True)
    assert st["embeds"].shape == (23, 16) and st["row_ids"].tolist() == list(range(100, 123))
