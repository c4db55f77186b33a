"""Mixture-of-experts: routing math, layer numerics against a per-token loop, expert parallelism against one
process (Gloo ranks), and a small MoE GPT that learns.  Mirrors the reference's tests/unit_tests/transformer/moe."""
import math

import pytest
import torch

from tests.dist_utils import run_distributed


def _cfg(**kw):
    from megatron_lm_b200.config import TransformerConfig
    base = dict(num_layers=2, hidden_size=16, num_attention_heads=4, ffn_hidden_size=32, moe_ffn_hidden_size=24,
                num_moe_experts=4, moe_router_topk=2, hidden_dropout=0.0, attention_dropout=0.0,
                gated_linear_unit=True, activation_func="silu", add_bias_linear=False, normalization="RMSNorm",
                use_cpu_initialization=True, moe_aux_loss_coeff=0.0)
    base.update(kw)
    return TransformerConfig(**base)


# ------------------------------------------------------------------------------------------------ routing math
@pytest.mark.parametrize("pre", [False, True])
def test_topk_softmax_matches_loop(pre):
    from megatron_lm_b200.models.moe import topk_softmax_with_capacity
    torch.manual_seed(0)
    lg = torch.randn(13, 6)
    probs, rmap, tpe = topk_softmax_with_capacity(lg, 2, use_pre_softmax=pre)
    for t in range(13):
        idx = torch.topk(lg[t], 2).indices
        want = torch.softmax(lg[t], -1)[idx] if pre else torch.softmax(lg[t][idx], -1)
        assert set(idx.tolist()) == set(torch.nonzero(rmap[t]).flatten().tolist())
        assert torch.allclose(probs[t][idx], want, atol=1e-6)
        assert probs[t].count_nonzero() == 2
    assert torch.equal(tpe, rmap.sum(0))
    if not pre:
        assert torch.allclose(probs.sum(-1), torch.ones(13), atol=1e-6)


def test_sigmoid_routing_with_bias_and_scaling():
    from megatron_lm_b200.models.moe import topk_softmax_with_capacity
    torch.manual_seed(1)
    lg = torch.randn(9, 8)
    bias = torch.zeros(8)
    bias[3] = 10.0                                   # always chosen, but its weight stays the unbiased score
    probs, rmap, _ = topk_softmax_with_capacity(lg, 2, score_function="sigmoid", expert_bias=bias, scaling_factor=2.5)
    assert rmap[:, 3].all()
    s = torch.sigmoid(lg)
    for t in range(9):
        idx = torch.nonzero(rmap[t]).flatten()
        want = s[t][idx] / s[t][idx].sum() * 2.5
        assert torch.allclose(probs[t][idx], want, atol=1e-6)


@pytest.mark.parametrize("policy", ["probs", "position"])
def test_capacity_drops_to_the_cap(policy):
    from megatron_lm_b200.models.moe import get_capacity, topk_softmax_with_capacity
    torch.manual_seed(2)
    T, E, k = 32, 4, 2
    lg = torch.randn(T, E)
    lg[:, 0] += 3.0                                  # expert 0 is over-subscribed
    cap = get_capacity(T * k, E, 0.5)
    probs, rmap, tpe_before = topk_softmax_with_capacity(lg, k, capacity_factor=0.5, drop_policy=policy)
    assert cap == math.ceil(T * k / E * 0.5)
    assert int(rmap.sum(0).max()) <= cap and int(tpe_before[0]) > cap
    assert (probs[~rmap] == 0).all()
    padded = topk_softmax_with_capacity(lg, k, capacity_factor=0.5, drop_policy=policy, pad_to_capacity=True)[1]
    assert (padded.sum(0) == cap).all()


def test_group_limited_topk_stays_inside_chosen_groups():
    from megatron_lm_b200.models.moe import topk_softmax_with_capacity
    torch.manual_seed(3)
    lg = torch.randn(20, 16)
    _, rmap, _ = topk_softmax_with_capacity(lg, 4, use_pre_softmax=True, num_groups=4, group_topk=2)
    groups_hit = rmap.view(20, 4, 4).any(-1).sum(-1)
    assert (rmap.sum(-1) == 4).all() and (groups_hit <= 2).all()


def test_aux_and_z_loss_values():
    from megatron_lm_b200.models.moe import switch_load_balancing_loss_func, z_loss_func
    T, E, k = 8, 4, 2
    probs = torch.full((T, E), 1.0 / E)
    tpe = torch.full((E,), T * k / E)
    # perfectly balanced: loss == coeff
    assert abs(float(switch_load_balancing_loss_func(probs, tpe, k, 0.01, T, E)) - 0.01) < 1e-8
    skew = torch.tensor([T * k, 0.0, 0.0, 0.0])
    p2 = torch.zeros(T, E)
    p2[:, 0] = 1.0
    assert float(switch_load_balancing_loss_func(p2, skew, k, 0.01, T, E)) > 0.03
    lg = torch.randn(5, 7)
    assert torch.allclose(z_loss_func(lg, 0.1), 0.1 * torch.logsumexp(lg, -1).square().mean())


def test_sinkhorn_balances_columns():
    from megatron_lm_b200.models.moe import sinkhorn
    torch.manual_seed(4)
    out = sinkhorn(torch.randn(16, 4))
    assert torch.allclose(out.sum(0), torch.full((4,), 0.25), atol=1e-2)
    assert torch.allclose(out.sum(1), torch.full((16,), 1 / 16), atol=1e-2)


def test_expert_bias_update_direction():
    from megatron_lm_b200.models.moe import get_updated_expert_bias
    new = get_updated_expert_bias(torch.tensor([10.0, 2.0, 6.0, 6.0]), torch.zeros(4), 0.1)
    assert new.tolist() == pytest.approx([-0.1, 0.1, 0.0, 0.0])


def test_permute_unpermute_roundtrip():
    from megatron_lm_b200.models.moe import permute, unpermute
    torch.manual_seed(5)
    x = torch.randn(10, 6)
    rmap = torch.zeros(10, 4, dtype=torch.bool)
    for t in range(10):
        rmap[t, torch.randperm(4)[:2]] = True
    p, idx = permute(x, rmap)
    assert p.shape[0] == 20
    # expert-major order: the first rows are expert 0's tokens in token order
    assert torch.equal(p[:int(rmap[:, 0].sum())], x[rmap[:, 0]])
    probs = torch.rand(10, 4) * rmap
    back = unpermute(p, idx, (10, 6), probs, rmap)
    assert torch.allclose(back, x * probs.sum(-1, keepdim=True), atol=1e-6)


# ------------------------------------------------------------------------------------------------ layer numerics
def _loop_moe(layer, x):
    """Per-token evaluation of the routed experts with the layer's own router."""
    import torch.nn.functional as F
    probs, rmap = layer.router(x)
    h = x.reshape(-1, x.shape[-1])
    out = torch.zeros_like(h)
    w1, w2 = layer.experts.weight1, layer.experts.weight2
    for t in range(h.shape[0]):
        for e in torch.nonzero(rmap[t]).flatten().tolist():
            a = h[t] @ w1[e].t()
            g, u = a.chunk(2, -1)
            out[t] += probs[t, e] * ((F.silu(g) * u) @ w2[e].t())
    return out.view_as(x)


@pytest.mark.parametrize("dispatcher", ["alltoall", "allgather"])
@pytest.mark.parametrize("grouped", [True, False])
def test_moe_layer_matches_token_loop(dispatcher, grouped):
    from megatron_lm_b200.models.moe import MoELayer
    torch.manual_seed(6)
    cfg = _cfg(moe_token_dispatcher_type=dispatcher, moe_grouped_gemm=grouped)
    layer = MoELayer(cfg, 1)
    x = torch.randn(5, 3, 16)
    y, _ = layer(x)
    if grouped:
        assert torch.allclose(y, _loop_moe(layer, x), atol=1e-5)
    else:
        assert y.shape == x.shape and torch.isfinite(y).all()


def test_shared_expert_is_added():
    from megatron_lm_b200.models.moe import MoELayer
    torch.manual_seed(7)
    cfg = _cfg(moe_shared_expert_intermediate_size=24, moe_grouped_gemm=True)
    layer = MoELayer(cfg, 1)
    x = torch.randn(4, 2, 16)
    y, _ = layer(x)
    assert torch.allclose(y - layer.shared_experts(x), _loop_moe(layer, x), atol=1e-5)


def test_aux_loss_reaches_router_weight_only_when_enabled():
    from megatron_lm_b200.models.moe import MoELayer, clear_aux_losses_tracker, get_moe_metrics
    torch.manual_seed(8)
    x = torch.randn(6, 2, 16)
    grads = {}
    for coeff in (0.0, 0.1):
        torch.manual_seed(9)
        layer = MoELayer(_cfg(moe_aux_loss_coeff=coeff, moe_grouped_gemm=True,
                              moe_router_load_balancing_type="aux_loss"), 1).train()
        clear_aux_losses_tracker()
        y, _ = layer(x)
        y.sum().backward()
        grads[coeff] = layer.router.weight.grad.clone()
        if coeff:
            assert float(get_moe_metrics()["load_balancing_loss"][0]) > 0
    assert not torch.allclose(grads[0.0], grads[0.1])


# ------------------------------------------------------------------------------------------------ expert parallel
def _ep_rank(rank, world, dispatcher, out_path):
    import torch.distributed as dist
    from megatron_lm_b200.models.moe import MoELayer
    from megatron_lm_b200.parallel import state
    state.initialize_model_parallel(expert_model_parallel_size=world)
    cfg = _cfg(expert_model_parallel_size=world, moe_token_dispatcher_type=dispatcher, moe_grouped_gemm=True)
    layer = MoELayer(cfg, 1)
    g = torch.Generator().manual_seed(11)
    W1 = 0.2 * torch.randn(4, 48, 16, generator=g)
    W2 = 0.2 * torch.randn(4, 16, 24, generator=g)
    Wr = torch.randn(4, 16, generator=g)
    X = torch.randn(8, 2, 16, generator=g)
    El = 4 // world
    with torch.no_grad():
        layer.experts.weight1.copy_(W1[rank * El:(rank + 1) * El])
        layer.experts.weight2.copy_(W2[rank * El:(rank + 1) * El])
        layer.router.weight.copy_(Wr)
    x = X[:, rank:rank + 1].clone().requires_grad_(True)          # each rank owns one sequence of the batch
    y, _ = layer(x)
    (y * y).sum().backward()
    torch.save({"y": y.detach(), "dx": x.grad, "dw1": layer.experts.weight1.grad, "dw2": layer.experts.weight2.grad,
                "dwr": layer.router.weight.grad}, f"{out_path}.{rank}")
    state.destroy_model_parallel()


@pytest.mark.parametrize("dispatcher", ["alltoall", "allgather"])
def test_expert_parallel_matches_single_process(tmp_path, dispatcher):
    from megatron_lm_b200.models.moe import MoELayer
    out = str(tmp_path / "ep")
    run_distributed(_ep_rank, 2, dispatcher, out)
    g = torch.Generator().manual_seed(11)
    W1 = 0.2 * torch.randn(4, 48, 16, generator=g)
    W2 = 0.2 * torch.randn(4, 16, 24, generator=g)
    Wr = torch.randn(4, 16, generator=g)
    X = torch.randn(8, 2, 16, generator=g)
    layer = MoELayer(_cfg(moe_grouped_gemm=True), 1)
    with torch.no_grad():
        layer.experts.weight1.copy_(W1)
        layer.experts.weight2.copy_(W2)
        layer.router.weight.copy_(Wr)
    x = X.clone().requires_grad_(True)
    y, _ = layer(x)
    (y * y).sum().backward()
    parts = [torch.load(f"{out}.{r}") for r in range(2)]
    for r in range(2):
        assert torch.allclose(parts[r]["y"], y[:, r:r + 1].detach(), atol=1e-5)
        assert torch.allclose(parts[r]["dx"], x.grad[:, r:r + 1], atol=1e-5)
        # an expert's weights live on one rank and see the tokens of every rank
        assert torch.allclose(parts[r]["dw1"], layer.experts.weight1.grad[2 * r:2 * r + 2], atol=1e-5)
        assert torch.allclose(parts[r]["dw2"], layer.experts.weight2.grad[2 * r:2 * r + 2], atol=1e-5)
    assert torch.allclose(parts[0]["dwr"] + parts[1]["dwr"], layer.router.weight.grad, atol=1e-5)


# ------------------------------------------------------------------------------------------------ model level
def test_moe_gpt_learns_and_tracks_aux_loss():
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.models.moe import clear_aux_losses_tracker, track_moe_metrics
    torch.manual_seed(12)
    cfg = _cfg(moe_aux_loss_coeff=0.01, moe_router_load_balancing_type="aux_loss", moe_grouped_gemm=True,
               moe_z_loss_coeff=1e-3)
    model = GPTModel(cfg, vocab_size=64, max_sequence_length=16, position_embedding_type="rope").train()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    data = torch.randint(0, 64, (4, 17))
    pos = torch.arange(16).unsqueeze(0).expand(4, 16)
    clear_aux_losses_tracker()
    losses = []
    for _ in range(25):
        opt.zero_grad()
        loss = model(data[:, :-1], pos, None, labels=data[:, 1:]).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] - 0.5
    m = track_moe_metrics(1.0, 1)
    assert m["load_balancing_loss"] > 0 and m["z_loss"] > 0


def _ep_training_rank(rank, world, ep, out_path):
    """GPT with experts trained for a few steps with clipping active; returns losses and gradient norms."""
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.training import setup_model_and_optimizer, train_step
    from tests.model_utils import reinit_by_global_name
    state.initialize_model_parallel(expert_model_parallel_size=ep)
    cfg = _cfg(num_layers=2, num_moe_experts=4, moe_router_topk=2, expert_model_parallel_size=ep,
               moe_ffn_hidden_size=32, moe_token_dispatcher_type="alltoall", moe_aux_loss_coeff=0.0,
               use_cpu_initialization=True)
    V, S, B, NMB = 64, 16, 2, 2

    def provider(pre_process=True, post_process=True, vp_stage=None):
        m = GPTModel(cfg, V, S, position_embedding_type="rope", share_embeddings_and_output_weights=False)
        reinit_by_global_name(m, cfg, std=0.3)                # large weights: the clip coefficient is < 1
        if ep > 1:
            # the two expert-parallel ranks must hold different experts for the test to mean anything
            with torch.no_grad():
                for name, p in m.named_parameters():
                    if not getattr(p, "allreduce", True):
                        p.mul_(1.0 + 0.5 * state.get_expert_model_parallel_rank())
        return m
    model, opt, _ = setup_model_and_optimizer(
        provider, cfg, OptimizerConfig(lr=1e-2, weight_decay=0.0, clip_grad=0.5),
        DistributedDataParallelConfig(grad_reduce_in_fp32=True))
    gen = torch.Generator().manual_seed(5)
    data = torch.randint(0, V, (3, NMB * B, S + 1), generator=gen)
    dp = state.get_data_parallel_world_size()
    dpr = state.get_data_parallel_rank()
    nmb = NMB // dp
    out = []
    for step in range(3):
        rows = data[step][dpr * nmb * B:(dpr + 1) * nmb * B]

        def it():
            for i in range(nmb):
                r = rows[i * B:(i + 1) * B]
                yield r[:, :-1], r[:, 1:]

        def fwd(itr, m):
            tok, lab = next(itr)
            o = m(tok, labels=lab)
            return o, (lambda x: (x.float().mean(), {"lm loss": x.float().mean().detach()}))
        l, _, gn, _ = train_step(fwd, it(), model, opt, None, cfg, num_microbatches=nmb, seq_length=S,
                                 micro_batch_size=B)
        out.append((float(l["lm loss"]), float(gn)))
    torch.save(out, f"{out_path}.{rank}")


def test_expert_parallel_grad_norm_is_global(tmp_path):
    """Without the distributed optimizer the expert gradients' squared norm must still be summed over the
    expert-parallel ranks: every rank then clips with the same coefficient and reports the same norm."""
    p = str(tmp_path / "ep2")
    run_distributed(_ep_training_rank, 2, 2, p)
    a, b = torch.load(p + ".0"), torch.load(p + ".1")
    for (la, ga), (lb, gb) in zip(a, b):
        assert ga == pytest.approx(gb, rel=1e-6), (a, b)     # one global norm on both expert-parallel ranks
    assert a[0][1] > 0.5                                       # clipping was active


# ------------------------------------------------------------------------------------------------ routing variants
def test_forced_load_balancing_spreads_tokens_and_keeps_gradients():
    """Random routing scores: even a router that prefers one expert sends every expert about its share, and the
    router weight still receives a gradient (reference: test_routers.py test_force_load_balancing)."""
    from megatron_lm_b200.models.moe import MoELayer
    torch.manual_seed(0)
    layer = MoELayer(_cfg(moe_router_force_load_balancing=True, moe_grouped_gemm=True), 1)
    with torch.no_grad():
        layer.router.weight.zero_()
        layer.router.weight[0] += 5.0                          # learnt preference: everything to expert 0
    x = torch.randn(64, 8, 16).abs()
    probs, rmap = layer.router(x)
    counts = rmap.sum(0).float()
    assert counts.min() > 0.6 * counts.mean() and counts.max() < 1.4 * counts.mean()
    layer(x)[0].sum().backward()
    assert layer.router.weight.grad is not None and layer.router.weight.grad.abs().sum() > 0
    plain = MoELayer(_cfg(moe_grouped_gemm=True), 1)
    with torch.no_grad():
        plain.router.weight.zero_()
        plain.router.weight[0] += 5.0
    assert plain.router(x)[1][:, 0].all()


def test_probabilities_applied_before_the_expert():
    from megatron_lm_b200.models.moe import MoELayer
    import torch.nn.functional as F
    with pytest.raises(ValueError):
        _cfg(moe_apply_probs_on_input=True)                    # needs top-1 routing
    torch.manual_seed(1)
    layer = MoELayer(_cfg(moe_apply_probs_on_input=True, moe_router_topk=1, moe_grouped_gemm=True,
                          moe_router_pre_softmax=True), 1)
    x = torch.randn(6, 2, 16)
    y, _ = layer(x)
    probs, rmap = layer.router(x)
    h = x.reshape(-1, 16)
    want = torch.zeros_like(h)
    for t in range(h.shape[0]):
        e = int(rmap[t].float().argmax())
        a = (probs[t, e] * h[t]) @ layer.experts.weight1[e].t()
        g, u = a.chunk(2, -1)
        want[t] = (F.silu(g) * u) @ layer.experts.weight2[e].t()
    assert torch.allclose(y.reshape(-1, 16), want, atol=1e-5)


def test_device_limited_routing_is_group_limited_routing():
    cfg = _cfg(num_moe_experts=8, moe_router_topk=2, moe_router_topk_limited_devices=1, expert_model_parallel_size=4)
    assert cfg.moe_router_num_groups == 4 and cfg.moe_router_group_topk == 1


def test_moe_layer_recompute_gives_the_same_gradients():
    from megatron_lm_b200.models.gpt import GPTModel
    grads = []
    for recompute in (False, True):
        torch.manual_seed(3)
        cfg = _cfg(moe_layer_recompute=recompute, moe_grouped_gemm=True)
        m = GPTModel(cfg, 32, 16, parallel_output=False, position_embedding_type="rope")
        assert m.decoder.layers[0].recompute_mlp == recompute
        ids = torch.randint(0, 32, (2, 16))
        m.train()
        m(ids, labels=ids).mean().backward()
        grads.append({n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None})
    assert grads[0].keys() == grads[1].keys()
    for k in grads[0]:
        assert torch.allclose(grads[0][k], grads[1][k], atol=1e-6), k
