"""--overlap-param-gather with the distributed optimizer: the chained, overlapped parameter gathers must give the
same training trajectory and the same weights (at checkpoint time, on every data-parallel rank) as gathering
everything right after the optimizer step - for a dense model and for one with an expert-parallel buffer."""
import pytest
import torch

from tests.dist_utils import run_distributed

V, S, B, STEPS = 64, 16, 2, 3


def _run(rank, world, overlap, moe, out_path):
    import torch.distributed as dist
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.training import evaluate, setup_model_and_optimizer, train_step
    from tests.model_utils import reinit_by_global_name
    ep = 2 if moe else 1
    state.initialize_model_parallel(expert_model_parallel_size=ep)
    kw = dict(num_layers=3, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
              attention_dropout=0.0, use_cpu_initialization=True, normalization="RMSNorm", gated_linear_unit=True,
              activation_func="silu", add_bias_linear=False)
    if moe:
        kw.update(num_moe_experts=4, moe_router_topk=2, expert_model_parallel_size=ep, moe_ffn_hidden_size=32,
                  moe_token_dispatcher_type="alltoall", moe_aux_loss_coeff=1e-2)
    cfg = TransformerConfig(**kw)

    def provider(pre_process=True, post_process=True, vp_stage=None):
        m = GPTModel(cfg, V, S, position_embedding_type="rope", share_embeddings_and_output_weights=False)
        reinit_by_global_name(m, cfg)
        return m
    # a small bucket size gives each buffer several buckets, so the chain has links
    dcfg = DistributedDataParallelConfig(grad_reduce_in_fp32=True, use_distributed_optimizer=True,
                                         overlap_grad_reduce=True, overlap_param_gather=overlap, bucket_size=4000)
    model, opt, _ = setup_model_and_optimizer(
        provider, cfg, OptimizerConfig(lr=5e-3, weight_decay=0.01, clip_grad=1.0, use_distributed_optimizer=True), dcfg)
    assert len(model[0].bucket_groups) > 2
    if moe:
        assert model[0].expert_buffers and model[0].expert_buffers[0].dp_size == 2
    gen = torch.Generator().manual_seed(5)
    data = torch.randint(0, V, (STEPS + 1, world * B, S + 1), generator=gen)
    dpr = state.get_data_parallel_rank()

    def fwd_for(step):
        def fwd(it, m):
            r = data[step][dpr * B:(dpr + 1) * B]
            out = m(r[:, :-1], labels=r[:, 1:])
            return out, (lambda o: (o.float().mean(), {"lm loss": o.float().mean().detach()}))
        return fwd
    losses = []
    for step in range(STEPS):
        l, _, gn, _ = train_step(fwd_for(step), None, model, opt, None, cfg, num_microbatches=1, seq_length=S,
                                 micro_batch_size=B)
        losses.append(float(l["lm loss"]))
    # what a checkpoint written now would hold: every rank's buffers, after the forced gather
    for m in model:
        m.force_param_sync()
    flat = torch.cat([b.param_data.float() for b in model[0].buffers + model[0].expert_buffers])
    for buf in model[0].buffers + model[0].expert_buffers:
        if buf.dp_size > 1:
            mine = buf.param_data.clone()
            gathered = [torch.empty_like(mine) for _ in range(buf.dp_size)]
            dist.all_gather(gathered, mine, group=buf.dp_group)
            for g in gathered:
                assert torch.equal(g, mine), "data-parallel replicas hold different weights after the forced gather"
    ev = evaluate(fwd_for(STEPS), None, model, cfg, eval_iters=1, num_microbatches=1, seq_length=S, micro_batch_size=B)
    torch.save({"losses": losses, "weights": flat, "eval": ev}, f"{out_path}.{rank}")


@pytest.mark.parametrize("moe", [False, True])
def test_overlapped_param_gather_matches_immediate_gather(tmp_path, moe):
    world = 4 if moe else 2
    a, b = str(tmp_path / "plain"), str(tmp_path / "overlap")
    run_distributed(_run, world, False, moe, a)
    run_distributed(_run, world, True, moe, b)
    for r in range(world):
        ra, rb = torch.load(f"{a}.{r}"), torch.load(f"{b}.{r}")
        assert ra["losses"] == pytest.approx(rb["losses"], rel=1e-6, abs=1e-7), (ra["losses"], rb["losses"])
        assert torch.equal(ra["weights"], rb["weights"])
        for k in ra["eval"]:
            assert ra["eval"][k] == pytest.approx(rb["eval"][k], rel=1e-6)
