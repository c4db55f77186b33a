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


def test_tensor_aware_state_dict_round_trip():
    """Tensors out (hollow, picklable structure), tensors back in, device moves, sharded leaves keep their placement
    and only main replicas carry data."""
    import pickle
    import pytest
    from megatron_lm_b200.checkpoint.sharded import ShardedTensor
    from megatron_lm_b200.checkpoint.tensor_aware import TensorAwareStateDict
    w = torch.arange(12.0).view(3, 4)
    main = ShardedTensor.from_rank_offsets("layer.w", torch.ones(2, 4), (0, 1, 2), replica_id=0)
    copy = ShardedTensor.from_rank_offsets("layer.b", torch.zeros(4), replica_id=(0, 0, 1))
    sd = {"iteration": 7, "model": {"w": w, "nested": [torch.zeros(2, dtype=torch.int64), "text"], "sh": main,
                                    "replica": copy}, "opt": ({"step": 3}, torch.full((2,), 5.0))}
    ta = TensorAwareStateDict.from_state_dict(sd)
    assert not ta.is_hollow and len(list(ta.tensors)) == 4 and ta.nbytes() == 12 * 4 + 2 * 8 + 8 * 4 + 2 * 4
    tensors = ta.pop_tensors()
    assert ta.is_hollow and tensors[0] is w
    blob = pickle.dumps(ta)                                     # the hollow form travels / is kept on the host
    assert len(blob) < 4000
    with pytest.raises(RuntimeError):
        ta.to_state_dict()
    with pytest.raises(ValueError):
        ta.insert_tensors(tensors[:-1])
    with pytest.raises(ValueError):
        ta.insert_tensors([tensors[0].view(4, 3)] + tensors[1:])
    other = pickle.loads(blob)
    other.init_tensors()
    for dst, src in zip(other.tensors, tensors):
        dst.copy_(src)
    back = other.to_state_dict()
    assert back["iteration"] == 7 and back["model"]["nested"][1] == "text" and back["opt"][0] == {"step": 3}
    assert torch.equal(back["model"]["w"], w) and torch.equal(back["opt"][1], torch.full((2,), 5.0))
    sh = back["model"]["sh"]
    assert isinstance(sh, ShardedTensor) and sh.global_offset == (2, 0) and torch.equal(sh.data, torch.ones(2, 4))
    assert back["model"]["replica"].data is None                # not the main replica: protected elsewhere
    keep_all = TensorAwareStateDict.from_state_dict(sd, remove_redundant_data=False)
    assert len(list(keep_all.tensors)) == 5
    ta.insert_tensors(tensors)
    ta.copy_tensors_to_cpu()
    assert all(t.device.type == "cpu" for t in ta.tensors) and next(iter(ta.tensors)) is not w
    ta.restore_tensor_device()
    assert torch.equal(ta.to_state_dict()["model"]["w"], w)
