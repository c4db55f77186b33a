"""Sharded-tensor factories and the fully parallel save assignment."""
import torch

from megatron_lm_b200.checkpoint import sharded as ds
from tests.dist_utils import run_distributed


def test_factory_roundtrip(tmp_path):
    w = torch.arange(24.0).view(6, 4)

    def build(key, t, rid):
        g, u = t.chunk(2, 0)
        return {"gate": ds.ShardedTensor.from_rank_offsets(key + ".gate", g.clone(), replica_id=rid),
                "up": ds.ShardedTensor.from_rank_offsets(key + ".up", u.clone(), replica_id=rid)}
    merge = lambda d: torch.cat((d["gate"], d["up"]), 0)
    sd = {"fc1": ds.ShardedTensorFactory("fc1", w, build, merge), "step": 3}
    ds.apply_factories(sd)
    ds.save(sd, str(tmp_path))
    req = {"fc1": ds.ShardedTensorFactory("fc1", torch.zeros(6, 4), build, merge)}
    fac = ds.apply_factories(req)
    out = ds.apply_factory_merges(ds.load(req, str(tmp_path)), fac)
    assert torch.equal(out["fc1"], w) and out["step"] == 3


def _worker(rank, world):
    import torch.distributed as dist
    sd = {f"t{i}": ds.ShardedTensor.from_rank_offsets(f"t{i}", torch.full((10 * (i + 1),), float(i)), replica_id=rank)
          for i in range(4)}
    n = ds.distribute_main_replicas(sd, dist.group.WORLD)
    mains = [k for k, v in sd.items() if v.is_main_replica()]
    every = [None] * world
    dist.all_gather_object(every, (mains, n))
    owned = sorted(k for m, _ in every for k in m)
    assert owned == ["t0", "t1", "t2", "t3"]                     # each tensor written exactly once
    assert abs(every[0][1] - every[1][1]) <= 40 * 4               # balanced within the largest tensor


def test_fully_parallel_assignment():
    run_distributed(_worker, 2)
