"""Tensor-parallel building blocks on Gloo ranks: the autograd mappings (forward collective / backward conjugate),
column- and row-parallel linear layers against a dense layer (with and without sequence parallelism), the
vocab-parallel embedding and cross entropy, and the data broadcast from TP rank 0.
Mirrors the reference's tests/unit_tests/tensor_parallel/*."""
import torch
import torch.nn.functional as F

from tests.dist_utils import run_distributed


def _cfg(tp, sp=False):
    from megatron_lm_b200.config import TransformerConfig
    return TransformerConfig(num_layers=1, hidden_size=16, num_attention_heads=4, tensor_model_parallel_size=tp,
                             sequence_parallel=sp, use_cpu_initialization=True, hidden_dropout=0.0,
                             attention_dropout=0.0)


def _mappings(rank, world):
    from megatron_lm_b200.parallel import mappings as M
    from megatron_lm_b200.parallel import state
    state.initialize_model_parallel(tensor_model_parallel_size=world)
    g = torch.Generator().manual_seed(0)
    full = torch.randn(4 * world, 3, 2 * world, generator=g)

    # copy: identity forward, all-reduce backward
    x = full.clone().requires_grad_()
    y = M.copy_to_tensor_model_parallel_region(x)
    (y * (rank + 1)).sum().backward()
    assert torch.equal(y, full) and torch.allclose(x.grad, torch.full_like(full, sum(range(1, world + 1))))

    # reduce: all-reduce forward, identity backward
    x = (full * (rank + 1)).requires_grad_()
    y = M.reduce_from_tensor_model_parallel_region(x)
    y.sum().backward()
    assert torch.allclose(y, full * sum(range(1, world + 1))) and torch.equal(x.grad, torch.ones_like(full))

    # scatter / gather along the last dim are each other's conjugates
    x = full.clone().requires_grad_()
    part = M.scatter_to_tensor_model_parallel_region(x)
    assert torch.equal(part, full[..., 2 * rank:2 * rank + 2])
    back = M.gather_from_tensor_model_parallel_region(part)
    assert torch.equal(back, full)
    (back * full).sum().backward()
    assert torch.allclose(x.grad[..., 2 * rank:2 * rank + 2], full[..., 2 * rank:2 * rank + 2])

    # sequence-parallel region: scatter first dim; gather with reduce-scatter backward; reduce-scatter forward
    x = full.clone().requires_grad_()
    sp = M.scatter_to_sequence_parallel_region(x)
    assert torch.equal(sp, full[4 * rank:4 * rank + 4])
    gathered = M.gather_from_sequence_parallel_region(sp)
    assert torch.equal(gathered, full)
    (gathered * (rank + 1)).sum().backward()                  # each rank's gradient of the gathered tensor differs
    # reduce-scatter sums the ranks' gradients per shard; the scatter's backward gathers the shards again
    assert torch.allclose(x.grad, torch.full_like(full, sum(range(1, world + 1))))
    x = (full * (rank + 1)).requires_grad_()
    rs = M.reduce_scatter_to_sequence_parallel_region(x)
    assert torch.allclose(rs, full[4 * rank:4 * rank + 4] * sum(range(1, world + 1)))
    rs.sum().backward()
    assert torch.equal(x.grad, torch.ones_like(full))          # all-gather of ones

    # sequence <-> head exchange round trip
    t = torch.randn(6, 8 * world, generator=g) + rank           # [tokens / tp, h], different on every rank
    hp = M.all_to_all_sp2hp(t)
    assert hp.shape == (6 * world, 8)
    assert torch.allclose(hp[6 * rank:6 * rank + 6], t[:, 8 * rank:8 * rank + 8])
    assert torch.allclose(M.all_to_all_hp2sp(hp), t)
    state.destroy_model_parallel()


def test_mappings_forward_and_backward():
    run_distributed(_mappings, 2)


def _linears(rank, world, sp):
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.layers import ColumnParallelLinear, RowParallelLinear
    state.initialize_model_parallel(tensor_model_parallel_size=world)
    cfg = _cfg(world, sp)
    g = torch.Generator().manual_seed(1)
    W1, b1 = torch.randn(24, 16, generator=g) * 0.2, torch.randn(24, generator=g) * 0.1
    W2, b2 = torch.randn(16, 24, generator=g) * 0.2, torch.randn(16, generator=g) * 0.1
    X = torch.randn(8, 2, 16, generator=g)                      # [s, b, h]
    col = ColumnParallelLinear(16, 24, config=cfg, init_method=cfg.init_method, bias=True, skip_bias_add=False)
    row = RowParallelLinear(24, 16, config=cfg, init_method=cfg.init_method, bias=True, skip_bias_add=True)
    n1 = 24 // world
    with torch.no_grad():
        col.weight.copy_(W1[rank * n1:(rank + 1) * n1]); col.bias.copy_(b1[rank * n1:(rank + 1) * n1])
        row.weight.copy_(W2[:, rank * n1:(rank + 1) * n1]); row.bias.copy_(b2)
    s_loc = 8 // world
    x = (X[rank * s_loc:(rank + 1) * s_loc] if sp else X).clone().requires_grad_()
    h, _ = col(x)
    y, bias = row(F.gelu(h))
    y = y + bias
    # dense reference
    Xd = X.clone().requires_grad_()
    W1d, W2d = W1.clone().requires_grad_(), W2.clone().requires_grad_()
    yd = F.linear(F.gelu(F.linear(Xd, W1d, b1)), W2d, b2)
    want = yd[rank * s_loc:(rank + 1) * s_loc] if sp else yd
    assert torch.allclose(y, want, atol=1e-5)
    (yd * yd).sum().backward()
    (y * y).sum().backward()
    assert torch.allclose(x.grad, Xd.grad[rank * s_loc:(rank + 1) * s_loc] if sp else Xd.grad, atol=1e-5)
    assert torch.allclose(col.weight.grad, W1d.grad[rank * n1:(rank + 1) * n1], atol=1e-5)
    assert torch.allclose(row.weight.grad, W2d.grad[:, rank * n1:(rank + 1) * n1], atol=1e-5)
    if sp:
        # the row bias sees only this rank's tokens: its gradient is partial and flagged for the SP all-reduce
        assert getattr(row.bias, "sequence_parallel", False)
    state.destroy_model_parallel()


def test_column_row_linear_match_dense():
    run_distributed(_linears, 2, False)


def test_column_row_linear_match_dense_sequence_parallel():
    run_distributed(_linears, 2, True)


def _embedding_and_ce(rank, world):
    from megatron_lm_b200.ops.core import cross_entropy
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.layers import VocabParallelEmbedding
    state.initialize_model_parallel(tensor_model_parallel_size=world)
    cfg = _cfg(world)
    g = torch.Generator().manual_seed(2)
    V, H = 20, 16
    table = torch.randn(V, H, generator=g)
    ids = torch.randint(0, V, (3, 7), generator=g)
    emb = VocabParallelEmbedding(V, H, init_method=cfg.init_method, config=cfg)
    per = V // world
    with torch.no_grad():
        emb.weight.copy_(table[rank * per:(rank + 1) * per])
    out = emb(ids)
    assert torch.allclose(out, table[ids], atol=1e-6)
    out.sum().backward()
    counts = torch.bincount(ids.flatten(), minlength=V).float()[rank * per:(rank + 1) * per]
    assert torch.allclose(emb.weight.grad, counts.unsqueeze(1).expand(per, H))

    logits = torch.randn(3, 7, V, generator=g)
    target = torch.randint(0, V, (3, 7), generator=g)
    for smoothing in (0.0, 0.1):
        mine = logits[..., rank * per:(rank + 1) * per].clone().requires_grad_()
        loss = cross_entropy(mine, target, vocab_start=rank * per, vocab_total=V, label_smoothing=smoothing,
                             group=state.get_tensor_model_parallel_group())
        ref_in = logits.clone().requires_grad_()
        ref = F.cross_entropy(ref_in.view(-1, V), target.view(-1), reduction="none", label_smoothing=smoothing).view(3, 7)
        assert loss.shape == target.shape and torch.allclose(loss, ref, atol=1e-5)
        loss.sum().backward()
        ref.sum().backward()
        assert torch.allclose(mine.grad, ref_in.grad[..., rank * per:(rank + 1) * per], atol=1e-5)
    state.destroy_model_parallel()


def test_vocab_parallel_embedding_and_cross_entropy():
    run_distributed(_embedding_and_ce, 2)


def _batch_broadcast(rank, world):
    from types import SimpleNamespace
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.batch import broadcast_data, get_batch_on_this_tp_rank
    state.initialize_model_parallel(tensor_model_parallel_size=world)
    data = None
    if rank == 0:
        data = {"tokens": torch.arange(12).view(2, 6), "labels": torch.arange(12).view(2, 6) + 1,
                "position_ids": torch.arange(6).repeat(2, 1), "loss_mask": torch.ones(2, 6) * 0.5}
    got = get_batch_on_this_tp_rank(iter([data]) if rank == 0 else None, SimpleNamespace())
    assert got["tokens"].tolist() == torch.arange(12).view(2, 6).tolist() and got["tokens"].dtype == torch.int64
    assert got["loss_mask"].dtype == torch.float32 and float(got["loss_mask"].sum()) == 6.0
    d2 = broadcast_data(["a", "b"], {"a": torch.ones(3, 2), "b": torch.zeros(5)} if rank == 0 else None, torch.float32)
    assert d2["a"].shape == (3, 2) and d2["b"].shape == (5,)
    state.destroy_model_parallel()


def test_batch_is_broadcast_from_tp_rank_zero():
    run_distributed(_batch_broadcast, 2)
