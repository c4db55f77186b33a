"""Vocab-parallel cross entropy with the peer-memory statistics exchange equals the all-reduce path."""
import os

import pytest
import torch

from tests.gpu_dist_utils import run_on_gpus

pytestmark = pytest.mark.gpu


def _worker(rank, world):
    import torch.distributed as dist
    from megatron_lm_b200.ops.core import cross_entropy
    torch.manual_seed(3)
    rows, V = 384, 1024
    full = (torch.randn(rows, V, device="cuda") * 3).bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda")
    vl = V // world
    res = {}
    for peer in ("0", "1"):
        os.environ["MLB_CE_PEER"] = peer
        lg = full[:, rank * vl:(rank + 1) * vl].clone().requires_grad_()
        for ls in (0.0, 0.1):
            loss = cross_entropy(lg, tgt, vocab_start=rank * vl, vocab_total=V, label_smoothing=ls,
                                 group=dist.group.WORLD, inplace_backward=False)
            g, = torch.autograd.grad(loss.sum(), lg)
            res[(peer, ls)] = (loss.detach().clone(), g.float())
    ref = torch.nn.functional.cross_entropy(full.float(), tgt, reduction="none")
    assert torch.allclose(res[("1", 0.0)][0], ref, atol=2e-3, rtol=2e-3)
    for ls in (0.0, 0.1):
        assert torch.allclose(res[("0", ls)][0], res[("1", ls)][0], atol=1e-4, rtol=1e-4)
        assert torch.allclose(res[("0", ls)][1], res[("1", ls)][1], atol=1e-3, rtol=1e-3)


def test_ce_peer_matches_allreduce():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_on_gpus(_worker, 2)
