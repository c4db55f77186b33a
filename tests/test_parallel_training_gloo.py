"""TP / SP / PP / VPP / DP(+ZeRO-1) on CPU Gloo ranks must reproduce the single-process training
trajectory of the same model (same weights via name-seeded init, same data)."""
import pytest
import torch

from tests.dist_utils import run_distributed

V, S, B, NMB, STEPS = 96, 16, 2, 4, 4


def _make_cfg(tp, pp, vpp, sp, kind):
    from megatron_lm_b200.config import TransformerConfig
    kw = dict(num_layers=4, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
              attention_dropout=0.0, tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
              virtual_pipeline_model_parallel_size=vpp, sequence_parallel=sp, use_cpu_initialization=True)
    if kind == "llama-dealloc":
        # stage outputs are dropped right after they are sent; backward runs from their grad_fn alone
        kind = "llama"
        kw.update(deallocate_pipeline_outputs=True)
    if kind in ("llama-defer", "gpt-defer"):
        # the output layer's weight-gradient GEMMs wait for the end of the pipeline (at most 2 queued at a time)
        kind = kind.split("-")[0]
        kw.update(defer_embedding_wgrad_compute=True, wgrad_deferral_limit=2)
    if kind == "moe":
        # a large balance-loss coefficient: a wrong scale of its gradient on an early stage moves the trajectory
        kw.update(normalization="RMSNorm", gated_linear_unit=True, activation_func="silu", add_bias_linear=False,
                  num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=32, moe_aux_loss_coeff=0.5,
                  moe_router_load_balancing_type="aux_loss", moe_token_dispatcher_type="alltoall")
    if kind == "llama":
        kw.update(normalization="RMSNorm", gated_linear_unit=True, activation_func="silu", add_bias_linear=False,
                  num_query_groups=2)
    return TransformerConfig(**kw)


def _run(rank, world, tp, pp, vpp, sp, dist_opt, kind, out_path):
    import torch.distributed as dist
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.training import setup_model_and_optimizer, train_step
    from tests.model_utils import reinit_by_global_name
    state.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                                    virtual_pipeline_model_parallel_size=vpp)
    cfg = _make_cfg(tp, pp, vpp, sp, kind)
    tied = kind.startswith("gpt")

    def provider(pre_process=True, post_process=True, vp_stage=None):
        m = GPTModel(cfg, V, S, pre_process=pre_process, post_process=post_process, vp_stage=vp_stage,
                     position_embedding_type="rope" if kind in ("llama", "moe", "llama-dealloc", "llama-defer")
                     else "learned_absolute",
                     share_embeddings_and_output_weights=tied)
        reinit_by_global_name(m, cfg)
        if tied and post_process and not pre_process:
            # the last stage's copy of the tied weight starts equal to the first stage's
            g = torch.Generator().manual_seed(__import__("tests.model_utils", fromlist=["_seed"])._seed(
                "embedding.word_embeddings.weight"))
            full = 0.05 * torch.randn(V, cfg.hidden_size, generator=g)
            per = V // tp
            r = state.get_tensor_model_parallel_rank()
            with torch.no_grad():
                m.output_layer.weight.copy_(full[r * per:(r + 1) * per])
        return m

    dp = world // (tp * pp)
    model, opt, _ = setup_model_and_optimizer(
        provider, cfg, OptimizerConfig(lr=5e-3, weight_decay=0.01, clip_grad=1.0, use_distributed_optimizer=dist_opt),
        DistributedDataParallelConfig(grad_reduce_in_fp32=True, use_distributed_optimizer=dist_opt,
                                      overlap_grad_reduce=dist_opt))
    gen = torch.Generator().manual_seed(5)
    data = torch.randint(0, V, (STEPS, NMB * B, S + 1), generator=gen)     # global batch per step
    dpr = state.get_data_parallel_rank()
    nmb_local = NMB // dp
    losses = []
    for step in range(STEPS):
        rows = data[step][dpr * nmb_local * B:(dpr + 1) * nmb_local * B]

        def gen_it():
            for i in range(nmb_local):
                r = rows[i * B:(i + 1) * B]
                yield r[:, :-1], r[:, 1:]
        its = [gen_it() for _ in model] if len(model) > 1 else gen_it()

        def fwd(it, m):
            tok, lab = next(it)
            out = m(tok, labels=lab)
            return out, (lambda o: (o.float().mean(), {"lm loss": o.float().mean().detach()}))
        l, skipped, gnorm, _ = train_step(fwd, its, model, opt, None, cfg, num_microbatches=nmb_local, seq_length=S,
                                          micro_batch_size=B)
        losses.append((float(l["lm loss"]) if l else None, float(gnorm)))
    last = state.is_pipeline_last_stage()
    if last and state.get_tensor_model_parallel_rank() == 0 and dpr == 0:
        torch.save(losses, out_path)


def _trajectory(tmp_path, world, tp=1, pp=1, vpp=None, sp=False, dist_opt=False, kind="llama"):
    out = str(tmp_path / f"traj_{world}_{tp}_{pp}_{vpp}_{sp}_{dist_opt}_{kind}.pt")
    run_distributed(_run, world, tp, pp, vpp, sp, dist_opt, kind, out)
    return torch.load(out)


def _close(a, b, tol=2e-4):
    for (la, ga), (lb, gb) in zip(a, b):
        assert abs(la - lb) < tol * max(1.0, abs(la)), (a, b)
        assert abs(ga - gb) < 5e-3 * max(1.0, abs(ga)), (a, b)


@pytest.fixture(scope="module")
def baseline(tmp_path_factory):
    d = tmp_path_factory.mktemp("base")
    return {k: _trajectory(d, 1, kind=k) for k in ("llama", "gpt")}


def test_baseline_learns(baseline):
    assert baseline["llama"][-1][0] < baseline["llama"][0][0]


@pytest.mark.parametrize("sp", [False, True])
def test_tensor_parallel_matches(tmp_path, baseline, sp):
    _close(_trajectory(tmp_path, 2, tp=2, sp=sp), baseline["llama"])


def test_tensor_parallel_gpt_tied_embeddings(tmp_path, baseline):
    _close(_trajectory(tmp_path, 2, tp=2, sp=True, kind="gpt"), baseline["gpt"])


def test_pipeline_parallel_matches(tmp_path, baseline):
    _close(_trajectory(tmp_path, 2, pp=2), baseline["llama"])


def test_pipeline_tied_embeddings_match(tmp_path, baseline):
    _close(_trajectory(tmp_path, 2, pp=2, kind="gpt"), baseline["gpt"])


def test_interleaved_pipeline_matches(tmp_path, baseline):
    _close(_trajectory(tmp_path, 2, pp=2, vpp=2), baseline["llama"])


def test_interleaved_pipeline_with_deallocated_outputs(tmp_path, baseline):
    _close(_trajectory(tmp_path, 2, pp=2, vpp=2, kind="llama-dealloc"), baseline["llama"])


@pytest.mark.parametrize("kind,vpp", [("llama", None), ("gpt", None), ("llama", 2)])
def test_deferred_output_layer_weight_gradient_matches(tmp_path, baseline, kind, vpp):
    from megatron_lm_b200.parallel import layers
    _close(_trajectory(tmp_path, 2, pp=2, vpp=vpp, kind=kind + "-defer"), baseline[kind])
    assert not layers._DEFERRED_WGRADS


def test_pipeline_parallel_moe_aux_loss_scale(tmp_path):
    """The load-balancing loss of MoE layers on the first pipeline stage gets the same gradient scale
    (1 / microbatches) as on the last stage: two stages reproduce the single-stage trajectory."""
    base = _trajectory(tmp_path, 1, kind="moe")
    _close(_trajectory(tmp_path, 2, pp=2, kind="moe"), base)


@pytest.mark.parametrize("dist_opt", [False, True])
def test_data_parallel_matches(tmp_path, baseline, dist_opt):
    _close(_trajectory(tmp_path, 2, dist_opt=dist_opt), baseline["llama"])


def test_tp2_pp2_sp_distopt(tmp_path, baseline):
    _close(_trajectory(tmp_path, 4, tp=2, pp=2, sp=True), baseline["llama"])


def test_tp4_pp2_vpp2_eight_ranks(tmp_path, baseline):
    """The 8-GPU layout of the headline benchmark (tensor 4 x pipeline 2 with 2 virtual stages, sequence parallel,
    distributed optimizer) on 8 Gloo ranks."""
    _close(baseline["gpt"], _trajectory(tmp_path, 8, tp=4, pp=2, vpp=2, sp=True, dist_opt=True, kind="gpt"))


def _run_cp(rank, world, cp, comm, out_path):
    """Context-parallel training: every rank holds its zig-zag slice of each sequence."""
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.context_parallel import zigzag_indices
    from megatron_lm_b200.training.training import setup_model_and_optimizer, train_step
    from tests.model_utils import reinit_by_global_name
    state.initialize_model_parallel(context_parallel_size=cp)
    cfg = _make_cfg(1, 1, None, False, "llama")
    cfg.context_parallel_size = cp
    cfg.cp_comm_type = comm

    def provider(pre_process=True, post_process=True, vp_stage=None):
        m = GPTModel(cfg, V, S, position_embedding_type="rope")
        reinit_by_global_name(m, cfg)
        return m
    model, opt, _ = setup_model_and_optimizer(provider, cfg, OptimizerConfig(lr=5e-3, weight_decay=0.01, clip_grad=1.0),
                                              DistributedDataParallelConfig(grad_reduce_in_fp32=True))
    gen = torch.Generator().manual_seed(5)
    data = torch.randint(0, V, (STEPS, NMB * B, S + 1), generator=gen)
    idx = zigzag_indices(S, cp, state.get_context_parallel_rank())
    losses = []
    for step in range(STEPS):
        def gen_it():
            for i in range(NMB):
                r = data[step][i * B:(i + 1) * B]
                yield r[:, :-1][:, idx], r[:, 1:][:, idx]
        it = gen_it()

        def fwd(it_, m):
            tok, lab = next(it_)
            out = m(tok, labels=lab)

            def lf(o):
                tot = torch.stack([o.float().sum(), torch.tensor(float(o.numel()))])
                torch.distributed.all_reduce(tot, group=state.get_context_parallel_group())
                # the gradient of the cp-summed loss w.r.t. local tokens is that of the local sum
                loss = o.float().sum() / tot[1]
                return loss * cp, {"lm loss": (tot[0] / tot[1]).detach()}
            return out, lf
        l, _, gn, _ = train_step(fwd, it, model, opt, None, cfg, num_microbatches=NMB, seq_length=S, micro_batch_size=B)
        losses.append((float(l["lm loss"]), float(gn)))
    if rank == 0:
        torch.save(losses, out_path)


@pytest.mark.parametrize("comm", ["p2p", "a2a", "all_gather"])
def test_context_parallel_matches(tmp_path, baseline, comm):
    out = str(tmp_path / f"cp_{comm}.pt")
    run_distributed(_run_cp, 2, 2, comm, out)
    _close(torch.load(out), baseline["llama"])


def _run_multi_instance(rank, world, instances, out_path):
    """Distributed optimizer with several instances: reduce-scatter inside an instance, all-reduce across."""
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.training import setup_model_and_optimizer, train_step
    from tests.model_utils import reinit_by_global_name
    state.initialize_model_parallel(num_distributed_optimizer_instances=instances)
    cfg = _make_cfg(1, 1, None, False, "llama")

    def provider(pre_process=True, post_process=True, vp_stage=None):
        m = GPTModel(cfg, V, S, position_embedding_type="rope")
        reinit_by_global_name(m, cfg)
        return m
    model, opt, _ = setup_model_and_optimizer(
        provider, cfg, OptimizerConfig(lr=5e-3, weight_decay=0.01, clip_grad=1.0, use_distributed_optimizer=True),
        DistributedDataParallelConfig(grad_reduce_in_fp32=True, use_distributed_optimizer=True, overlap_grad_reduce=True,
                                      num_distributed_optimizer_instances=instances, bucket_size=5000))
    if instances > 1:
        assert model[0].buffers[0].dp_size == world // instances and model[0].buffers[0].inter_group is not None
    gen = torch.Generator().manual_seed(5)
    data = torch.randint(0, V, (STEPS, NMB * B, S + 1), generator=gen)
    nmb_local = NMB // world
    losses = []
    for step in range(STEPS):
        rows = data[step][rank * nmb_local * B:(rank + 1) * nmb_local * B]

        def gen_it():
            for i in range(nmb_local):
                r = rows[i * B:(i + 1) * B]
                yield r[:, :-1], r[:, 1:]

        def fwd(it, m):
            tok, lab = next(it)
            out = m(tok, labels=lab)
            return out, (lambda o: (o.float().mean(), {"lm loss": o.float().mean().detach()}))
        l, _, gnorm, _ = train_step(fwd, gen_it(), model, opt, None, cfg, num_microbatches=nmb_local, seq_length=S,
                                    micro_batch_size=B)
        losses.append((float(l["lm loss"]), float(gnorm)))
    if rank == 0:
        torch.save(losses, out_path)


def test_two_distributed_optimizer_instances_match(tmp_path, baseline):
    out = str(tmp_path / "inst2.pt")
    run_distributed(_run_multi_instance, 4, 2, out)
    _close(torch.load(out), baseline["llama"])
