"""C++ index builders against straightforward Python restatements."""
import numpy as np

from megatron_lm_b200.data import helpers as h


def _py_sample_idx(sizes, doc_idx, seq, n_samples, extra):
    out = [(0, 0)]
    pos, off = 0, 0
    for _ in range(n_samples):
        need = seq + extra
        while need > 0:
            avail = sizes[doc_idx[pos]] - off
            if avail >= need:
                off += need - extra
                need = 0
            else:
                need -= avail
                if pos == len(doc_idx) - 1:
                    off = sizes[doc_idx[pos]] - extra
                    need = 0
                else:
                    pos += 1
                    off = 0
        out.append((pos, off))
    return np.array(out, dtype=np.int64)


def test_sample_idx_matches_python():
    rng = np.random.default_rng(0)
    for _ in range(25):
        nd = int(rng.integers(3, 30))
        sizes = rng.integers(1, 40, nd).astype(np.int32)
        epochs = int(rng.integers(1, 4))
        doc = np.concatenate([rng.permutation(nd) for _ in range(epochs)]).astype(np.int32)
        seq = int(rng.integers(2, 25))
        tpe = int(sizes.sum())
        for extra in (0, 1):
            got = h.build_sample_idx(sizes, doc, seq, epochs, tpe, True, extra)
            n = (epochs * tpe - extra) // seq
            assert got.shape == (n + 1, 2)
            assert np.array_equal(got, _py_sample_idx(sizes, doc, seq, n, extra))


def test_sample_idx_covers_exact_token_spans():
    sizes = np.array([5, 3, 10, 2], dtype=np.int32)
    doc = np.array([0, 1, 2, 3, 2, 0, 1, 3], dtype=np.int32)
    idx = h.build_sample_idx(sizes, doc, 4, 2, 20, True, 1)
    stream = np.concatenate([np.arange(sizes[d]) + 100 * d for d in doc])
    starts = np.cumsum([0] + [sizes[d] for d in doc])
    for i in range(len(idx) - 1):
        a = starts[idx[i, 0]] + idx[i, 1]
        b = starts[idx[i + 1, 0]] + idx[i + 1, 1]
        assert b - a == 4                      # consecutive samples share the extra token
        assert len(stream[a:b + 1]) == 5


def test_blending_tracks_weights():
    di, dsi = h.build_blending_indices([0.5, 0.3, 0.2], 1000)
    counts = np.bincount(di, minlength=3)
    assert abs(counts[0] - 500) <= 1 and abs(counts[1] - 300) <= 1 and abs(counts[2] - 200) <= 1
    for d in range(3):                             # per-dataset sample ids are 0,1,2,... in order
        assert np.array_equal(dsi[di == d], np.arange(counts[d]))


def test_exhaustive_blending_uses_everything_once():
    sizes = [30, 10, 25]
    di, dsi = h.build_exhaustive_blending_indices(sizes)
    assert len(di) == 65
    for d, n in enumerate(sizes):
        assert np.array_equal(np.sort(dsi[di == d]), np.arange(n))


def test_bert_and_block_mappings_are_consistent():
    rng = np.random.default_rng(1)
    n_docs = 50
    sent_per_doc = rng.integers(1, 12, n_docs)
    docs = np.concatenate([[0], np.cumsum(sent_per_doc)]).astype(np.int64)
    sizes = rng.integers(5, 60, docs[-1]).astype(np.int32)
    m = h.build_mapping(docs, sizes, 2, 10_000, 128, 0.1, 1234, 2)
    assert m.shape[1] == 3 and len(m) > 0
    assert np.all(m[:, 1] > m[:, 0]) and np.all(m[:, 2] <= 128) and np.all(m[:, 2] >= 2)
    for a, b, _ in m[:50]:                         # a sample never crosses a document boundary
        d = np.searchsorted(docs, a, side="right") - 1
        assert b <= docs[d + 1]
    titles = rng.integers(1, 8, n_docs).astype(np.int32)
    bm = h.build_blocks_mapping(docs, sizes, titles, 1, 10_000, 128, 1234, False)
    assert bm.shape[1] == 4 and len(np.unique(bm[:, 3])) == len(bm)
