"""ZeRO-3 sharded data parallelism on 2 GPUs (NCCL all-gather / reduce-scatter, bf16 weights, CUDA kernels) follows
the same loss trajectory as the unsharded strategy."""
import pytest
import torch

from tests.gpu_dist_utils import run_on_gpus

pytestmark = pytest.mark.gpu


def _worker(rank, world, out_path):
    import contextlib
    import torch.distributed as dist
    from megatron_lm_b200.config import DistributedDataParallelConfig, TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.parallel.fsdp import FullyShardedDataParallel, ShardedAdam
    res = {}
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, 256, (3, world, 2, 65), generator=g).cuda()
    for strategy in ("no_shard", "optim_grads_params"):
        torch.manual_seed(1)
        cfg = TransformerConfig(num_layers=2, hidden_size=128, num_attention_heads=2, ffn_hidden_size=256,
                                hidden_dropout=0.0, attention_dropout=0.0, add_bias_linear=False, kv_channels=64,
                                normalization="RMSNorm", gated_linear_unit=True, params_dtype=torch.bfloat16, bf16=True,
                                use_cpu_initialization=False)
        m = GPTModel(cfg, 256, 64, position_embedding_type="rope").cuda()
        f = FullyShardedDataParallel(cfg, DistributedDataParallelConfig(data_parallel_sharding_strategy=strategy), m,
                                     group=dist.group.WORLD)
        opt = ShardedAdam([f], lr=1e-3, weight_decay=0.01, clip_grad=1.0)
        losses = []
        for s in range(3):
            f.zero_grad_buffer()
            loss = f(data[s, rank][:, :-1], labels=data[s, rank][:, 1:]).float().mean()
            loss.backward()
            opt.step()
            t = loss.detach().clone()
            dist.all_reduce(t)
            losses.append(float(t) / world)
        res[strategy] = losses
        if strategy == "optim_grads_params":
            assert all(p.untyped_storage().size() == 0 for p in m.decoder.layers[0].parameters())
    for a, b in zip(res["no_shard"], res["optim_grads_params"]):
        assert abs(a - b) < 5e-3, res
    assert res["no_shard"][-1] < res["no_shard"][0]


def test_zero3_matches_unsharded_on_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_on_gpus(_worker, 2, str(tmp_path / "x"))
