"""Sharded data parallelism (every strategy) on 2 Gloo ranks equals single-process AdamW training."""
import pytest
import torch

from tests.dist_utils import run_distributed


def _build(seed=3):
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    torch.manual_seed(seed)
    cfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, add_bias_linear=True)
    return cfg, GPTModel(cfg, 64, 16)


def _reference(steps, batches):
    cfg, m = _build()
    decay = [p for p in m.parameters() if p.dim() > 1]
    nodecay = [p for p in m.parameters() if p.dim() <= 1]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": nodecay, "weight_decay": 0.0}],
                            lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    losses = []
    for s in range(steps):
        opt.zero_grad()
        tot = 0.0
        for ids in batches[s]:
            loss = m(ids, labels=ids).mean() / len(batches[s])
            loss.backward()
            tot += float(loss)
        for p in m.parameters():                      # ops deliver through .grad when there is no main_grad
            assert p.grad is not None
        torch.nn.utils.clip_grad_norm_(m.parameters(), 1.0)
        opt.step()
        losses.append(tot)
    return losses, {k: v.detach().clone() for k, v in m.state_dict().items()}


def _worker(rank, world, strategy):
    import torch.distributed as dist
    from megatron_lm_b200.config import DistributedDataParallelConfig
    from megatron_lm_b200.parallel.fsdp import FullyShardedDataParallel, ShardedAdam
    g = torch.Generator().manual_seed(11)
    batches = [[torch.randint(0, 64, (2, 12), generator=g) for _ in range(4)] for _ in range(3)]
    ref_losses, ref_sd = _reference(3, batches)
    cfg, m = _build()
    dcfg = DistributedDataParallelConfig(data_parallel_sharding_strategy=strategy)
    f = FullyShardedDataParallel(cfg, dcfg, m, group=dist.group.WORLD)
    opt = ShardedAdam([f], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, clip_grad=1.0)
    for s in range(3):
        f.zero_grad_buffer()
        mine = batches[s][rank::world]               # 2 microbatches per rank
        tot = torch.zeros(1)
        for i, ids in enumerate(mine):
            last = i == len(mine) - 1
            ctx = f.no_sync() if not last else __import__("contextlib").nullcontext()
            with ctx:
                loss = f(ids, labels=ids).mean() / len(mine)
                loss.backward()
            tot += loss.detach()
        opt.step()
        dist.all_reduce(tot)
        assert abs(float(tot) / world - ref_losses[s]) < 2e-4, (s, float(tot) / world, ref_losses[s])
    sd = f.state_dict()
    for k, v in ref_sd.items():
        assert torch.allclose(sd[k], v, atol=2e-4, rtol=1e-3), (k, (sd[k] - v).abs().max())
    if strategy == "optim_grads_params":
        assert all(p.untyped_storage().size() == 0 for p in m.decoder.layers[0].parameters())      # weights are dropped between uses


@pytest.mark.parametrize("strategy", ["no_shard", "optim", "optim_grads", "optim_grads_params"])
def test_fsdp_matches_single_process(strategy):
    run_distributed(_worker, 2, strategy)
