"""Retro: retrieval cross-attention is causal at chunk granularity and trains."""
import torch

from megatron_lm_b200.models.retro import RetroConfig, RetroModel, get_retro_decoder_layer_numbers


def test_layer_numbers():
    assert get_retro_decoder_layer_numbers(12) == [6, 9, 12]
    assert get_retro_decoder_layer_numbers(24) == [9, 12, 15, 18, 21, 24]


def test_retro_causality_and_grad():
    torch.manual_seed(0)
    cfg = RetroConfig(num_layers=6, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                      attention_dropout=0.0, retro_chunk_length=4, retro_num_neighbors=2, retro_num_retrieved_chunks=2,
                      retro_encoder_num_layers=1, retro_encoder_hidden_dropout=0.0, retro_encoder_attention_dropout=0.0)
    m = RetroModel(cfg, 64, 32).eval()
    ids = torch.randint(0, 64, (2, 12))
    ctx = torch.randint(0, 64, (2, 3, 2, 8))
    with torch.no_grad():
        a = m(ids, context_input_ids=ctx)
        # neighbours of the last chunk influence nothing before the last token of that chunk
        ctx2 = ctx.clone(); ctx2[:, 2] = 1
        b = m(ids, context_input_ids=ctx2)
        # future tokens do not influence earlier positions
        ids3 = ids.clone(); ids3[:, 8:] = 2
        c = m(ids3, context_input_ids=ctx)
    assert a.shape == (2, 12, 64)
    assert torch.allclose(a[:, :11], b[:, :11], atol=1e-5) and not torch.allclose(a[:, 11], b[:, 11], atol=1e-5)
    assert torch.allclose(a[:, :7], c[:, :7], atol=1e-5)
    m.train()
    m(ids, context_input_ids=ctx, labels=ids).mean().backward()
    p = m.retro_layers["6"].attn.linear_q.weight
    g = p.grad if p.grad is not None else p.main_grad
    assert g.abs().sum() > 0
    # a closed gate takes the retrieval out: the neighbours no longer matter
    cfg.retro_attention_gate = 0.0
    m.eval()
    with torch.no_grad():
        assert torch.allclose(m(ids, context_input_ids=ctx), m(ids, context_input_ids=ctx2), atol=1e-6)


def _corpus(tmp_path, ndocs=12, seed=0):
    import numpy as np
    from megatron_lm_b200.data.indexed_dataset import IndexedDataset, IndexedDatasetBuilder, get_bin_path, get_idx_path
    prefix = str(tmp_path / "corpus")
    b = IndexedDatasetBuilder(get_bin_path(prefix), dtype=np.int32)
    rng = np.random.RandomState(seed)
    docs = []
    for d in range(ndocs):
        # documents come in topical pairs: 2d and 2d+1 draw from the same narrow token range
        lo = 10 + 20 * (d // 2)
        toks = rng.randint(lo, lo + 20, size=rng.randint(40, 70)).tolist()
        docs.append(toks)
        b.add_item(toks)
        b.end_document()
    b.finalize(get_idx_path(prefix))
    return IndexedDataset(prefix), docs, prefix


def test_chunk_db_embeddings_neighbours_and_dataset(tmp_path):
    import numpy as np
    import torch
    from megatron_lm_b200.data import retro_preprocess as R
    ds, docs, prefix = _corpus(tmp_path)
    db = R.build_chunk_db(ds, chunk_length=8)
    assert len(db) == sum((len(d) + 7) // 8 for d in docs)
    c = 5
    d, o, ln = int(db.doc_ids[c]), int(db.offsets[c]), int(db.lengths[c])
    assert R.chunk_tokens(ds, db, [c])[0, :ln].tolist() == docs[d][o:o + ln]
    db.save(str(tmp_path / "db.npz"))
    assert (R.ChunkDB.load(str(tmp_path / "db.npz")).offsets == db.offsets).all()
    table = torch.nn.functional.one_hot(torch.arange(200), 200).float()         # bag-of-tokens embedding
    emb = R.embed_chunks(ds, db, R.mean_pool_embedder(table))
    assert emb.shape == (len(db), 200) and torch.allclose(emb.norm(dim=-1), torch.ones(len(db)), atol=1e-5)
    nb = R.query_neighbors(emb, emb, 2, db.doc_ids, db.doc_ids)
    assert nb.shape == (len(db), 2) and (nb >= 0).all()
    assert (db.doc_ids[nb] != db.doc_ids[:, None]).all()                       # never the query's own document
    # the nearest neighbour of most chunks lies in the topical twin of its document
    twin = (db.doc_ids[nb[:, 0]] // 2) == (db.doc_ids // 2)
    assert twin.mean() > 0.9
    # brute-force check of one row
    sim = emb[7] @ emb.t()
    sim[torch.as_tensor(db.doc_ids == db.doc_ids[7])] = -1e9
    assert int(sim.argmax()) == int(nb[7, 0])
    rd = R.RetroDataset(ds, db, nb, sample_length=32, num_neighbors=2)
    assert len(rd) > 0
    s = rd[0]
    assert s["text"].shape == (32,) and s["neighbor_tokens"].shape == (4, 2, 16)
    c0 = int(rd.starts[0])
    first = int(nb[c0, 0])
    assert s["neighbor_tokens"][0, 0, :8].tolist() == R.chunk_tokens(ds, db, [first])[0].tolist()


def test_retro_preprocess_cli_and_model_step(tmp_path):
    import numpy as np
    import torch
    from megatron_lm_b200.data import retro_preprocess as R
    from megatron_lm_b200.models.retro import RetroConfig, RetroModel
    ds, docs, prefix = _corpus(tmp_path, ndocs=8, seed=1)
    out = str(tmp_path / "retro")
    R.main(["--input", prefix, "--output", out, "--chunk-length", "8", "--num-neighbors", "2", "--vocab-size", "200",
            "--embed-dim", "32", "--device", "cpu"])
    db = R.ChunkDB.load(out + "/chunk_db.npz")
    nb = np.load(out + "/neighbors.npy")
    assert nb.shape == (len(db), 2) and torch.load(out + "/embeddings.pt").shape == (len(db), 32)
    rd = R.RetroDataset(ds, db, nb, sample_length=16, num_neighbors=2)
    batch = [rd[i] for i in range(2)]
    text = torch.stack([b["text"] for b in batch])
    ctx = torch.stack([b["neighbor_tokens"] for b in batch])                   # [b, l, k, r]
    cfg = RetroConfig(num_layers=6, hidden_size=32, num_attention_heads=4, use_cpu_initialization=True,
                      hidden_dropout=0.0, attention_dropout=0.0, retro_chunk_length=8, retro_retrieved_length=16,
                      retro_num_neighbors=2)
    m = RetroModel(cfg, 256, 64)
    loss = m(text[:, :-1] if False else text, context_input_ids=ctx, labels=text).float().mean()
    loss.backward()
    assert torch.isfinite(loss)
