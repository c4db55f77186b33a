"""Distributed optimizer with peer-memory collectives (gradient pull-reduce, AdamW storing into every rank's
parameter buffer) equals the NCCL reduce-scatter / all-gather path on 2 data-parallel GPUs."""
import pytest
import torch

from tests.gpu_dist_utils import run_on_gpus

pytestmark = pytest.mark.gpu


def _train(rank, world, peer, out_path, overlap=False):
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.ops import _lib
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.training import setup_model_and_optimizer, train_step
    from tests.model_utils import reinit_by_global_name
    state.initialize_model_parallel(create_gloo_process_groups=False)
    V, S, B = 512, 256, 1
    cfg = TransformerConfig(num_layers=2, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512,
                            normalization="RMSNorm", gated_linear_unit=True, activation_func="silu",
                            add_bias_linear=False, hidden_dropout=0.0, attention_dropout=0.0, bf16=True,
                            params_dtype=torch.bfloat16, kv_channels=64)

    def provider(pre_process=True, post_process=True, vp_stage=None):
        m = GPTModel(cfg, V, S, position_embedding_type="rope")
        reinit_by_global_name(m, cfg, std=0.02)
        return m
    dcfg = DistributedDataParallelConfig(grad_reduce_in_fp32=True, use_distributed_optimizer=True,
                                         peer_memory_collectives=peer, bucket_size=200000,
                                         overlap_grad_reduce=overlap)
    model, opt, _ = setup_model_and_optimizer(provider, cfg, OptimizerConfig(lr=1e-3, clip_grad=1.0, bf16=True,
                                                                             use_distributed_optimizer=True), dcfg)
    assert (model[0].buffers[0].peer is not None) == peer
    g = torch.Generator().manual_seed(11)
    data = torch.randint(0, V, (4, world, B, S + 1), generator=g).cuda()
    losses = []
    for step in range(4):
        def fwd(it, m):
            out = m(data[step, rank][:, :-1], labels=data[step, rank][:, 1:])
            return out, (lambda o: (o.float().mean(), {"lm loss": o.float().mean().detach()}))
        l, _, gn, _ = train_step(fwd, None, model, opt, None, cfg, num_microbatches=1, seq_length=S, micro_batch_size=B)
        losses.append((float(l["lm loss"]), float(gn)))
    torch.cuda.synchronize()
    _lib.check_status()
    if rank == 0:
        torch.save({"losses": losses, "w": model[0].module.decoder.layers[1].mlp.linear_fc2.weight.detach().float().cpu()},
                   out_path)


@pytest.mark.parametrize("overlap", [False, True])
def test_peer_collectives_match_nccl(tmp_path, overlap):
    """``overlap``: every bucket's pull is launched on the side stream as soon as the bucket is complete locally and
    waits in the kernel for the peers' readiness words, while the backward pass goes on."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    a, b = str(tmp_path / "nccl.pt"), str(tmp_path / "peer.pt")
    run_on_gpus(_train, 2, False, a, overlap)
    run_on_gpus(_train, 2, True, b, overlap)
    ra, rb = torch.load(a), torch.load(b)
    for (la, ga), (lb, gb) in zip(ra["losses"], rb["losses"]):
        assert abs(la - lb) < 2e-3 and abs(ga - gb) < 2e-3 * max(1.0, ga), (ra["losses"], rb["losses"])
    assert torch.allclose(ra["w"], rb["w"], atol=1e-3, rtol=1e-2)
