"""A rank that raises makes every rank abandon the attempt and run the function again in the same processes."""
import os
from datetime import timedelta

import torch

from tests.dist_utils import _free_port


def _proc(rank, world, port, q):
    import torch.distributed as dist
    from megatron_lm_b200.training.inprocess_restart import RestartWrapper
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=30))
    w = RestartWrapper(store, rank, world, max_restarts=2, barrier_timeout=30)

    def train(wrapper, attempt):
        dist.init_process_group("gloo", store=dist.PrefixStore(f"pg{attempt}", store), rank=rank, world_size=world,
                                timeout=timedelta(seconds=10))
        total = 0.0
        for step in range(4):
            wrapper.check()
            if attempt == 0 and rank == 1 and step == 2:
                raise ValueError("injected host-side failure")
            t = torch.ones(1) * (rank + 1)
            try:
                dist.all_reduce(t)
            except RuntimeError as e:                      # the failed rank never joins: the collective errors out
                from megatron_lm_b200.training.inprocess_restart import RestartSignal
                raise RestartSignal(str(e))
            total += float(t)
        dist.destroy_process_group()
        return attempt, total
    q.put((rank, w.run(train)))


def test_restart_after_injected_failure():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    ps = [ctx.Process(target=_proc, args=(r, 2, port, q), daemon=True) for r in range(2)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(90)
        assert not p.is_alive() and p.exitcode == 0
    res = dict(q.get() for _ in range(2))
    assert res[0] == (1, 12.0) and res[1] == (1, 12.0)          # second attempt, 4 steps x (1 + 2)
