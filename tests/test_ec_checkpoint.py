"""Erasure-coded in-memory checkpoint: field math, placement, and multi-rank (Gloo) save / lose / rebuild."""
import itertools

import numpy as np
import pytest
import torch

from megatron_lm_b200.checkpoint import gf256
from megatron_lm_b200.checkpoint.ec_plan import plan_stripes
from tests.dist_utils import run_distributed


def test_field_axioms():
    _, _, mul = gf256.tables()
    assert all(gf256.gf_mul(a, gf256.gf_inv(a)) == 1 for a in range(1, 256))
    assert np.array_equal(mul, mul.T)
    a, b, c = 87, 201, 13
    assert gf256.gf_mul(a, b ^ c) == gf256.gf_mul(a, b) ^ gf256.gf_mul(a, c)
    assert gf256.gf_mul(2, 0x80) == 0x1D                     # reduction by x^8+x^4+x^3+x^2+1


@pytest.mark.parametrize("k,m", [(2, 1), (6, 2), (4, 3), (5, 4)])
def test_every_erasure_pattern_decodes(k, m):
    rng = np.random.default_rng(0)
    data = [rng.integers(0, 256, 257, dtype=np.uint8) for _ in range(k)]
    members = data + gf256.apply_matrix_numpy(gf256.generator_matrix(k, m), data)
    for lost in itertools.combinations(range(k + m), m):
        present = [i for i in range(k + m) if i not in lost]
        M, use = gf256.decode_matrix(k, m, present, list(lost))
        rec = gf256.apply_matrix_numpy(M, [members[u] for u in use])
        for w, r in zip(lost, rec):
            assert np.array_equal(members[w], r)


@pytest.mark.parametrize("n,k,m,c", [(8, 6, 2, 12), (8, 6, 2, 7), (4, 2, 1, 9), (8, 3, 2, 4), (2, 2, 1, 5)])
def test_placement_never_colocates(n, k, m, c):
    plan = plan_stripes(n, k, m, c)
    plan.validate()
    for lost in itertools.combinations(range(n), min(m, n - 1) if not plan.stripes[0].host_only else 1):
        for s in plan.stripes:
            gone = sum(r in lost for r, _ in s.data)
            if not s.host_only:
                gone += sum(o in lost for o in s.parity_owners)
            assert gone <= m


def _save_lose_recover(rank, world, k, m, lost, chunk):
    from megatron_lm_b200.checkpoint.ec_checkpoint import ECCheckpointManager
    torch.manual_seed(100 + rank)
    state = [torch.randn(3000 + 17 * rank), torch.randn(50, 40), torch.randint(0, 100, (333,), dtype=torch.int32)]
    ref = [t.clone() for t in state]
    mgr = ECCheckpointManager(k=k, m=m, chunk_bytes=chunk)
    mgr.save(state, iteration=7)
    for t in state:                              # training moves on after the checkpoint
        t.add_(1) if t.is_floating_point() else t.add_(1)
    if rank in lost:
        mgr.drop_local_state()
        for t in state:
            t.zero_()
    it = mgr.recover(lost, tensors_out=state)
    assert it == 7
    for a, b in zip(state, ref):
        assert torch.equal(a, b), f"rank {rank} did not get back its bytes"


# the last case is the 8-rank Reed-Solomon k=6, m=2 layout with two ranks lost at once
# (4, 1, 2): one data member and two parity members per stripe - what --replication --replication-factor 3 asks for
@pytest.mark.parametrize("world,k,m,lost", [(2, 2, 1, [1]), (4, 3, 1, [2]), (4, 2, 2, [0, 3]), (4, 2, 1, [1]),
                                            (4, 1, 2, [1, 2]), (8, 6, 2, [2, 5])])
def test_save_lose_recover_gloo(world, k, m, lost):
    run_distributed(_save_lose_recover, world, k, m, lost, 4096)


def _state_dict_rank(rank, world):
    from megatron_lm_b200.checkpoint.ec_checkpoint import ECCheckpointManager
    from megatron_lm_b200.checkpoint.tensor_aware import TensorAwareStateDict
    torch.manual_seed(10 + rank)

    def fresh():
        return {"iteration": 0, "model": {"w": torch.randn(40, 30), "b": torch.randn(30)},
                "optimizer": {"state": [torch.randn(1200), torch.randn(1200)], "step": 0}}
    sd = fresh()
    sd["iteration"], sd["optimizer"]["step"] = 9, 9
    ref = {"w": sd["model"]["w"].clone(), "m": sd["optimizer"]["state"][1].clone()}
    mgr = ECCheckpointManager(k=1, m=1, chunk_bytes=2048)
    mgr.save_state_dict(sd, iteration=9)
    sd["model"]["w"].add_(1.0)
    if rank == 1:
        # a replacement process: nothing in memory, structure from a freshly built state dict
        mgr.drop_local_state()
        mgr.hollow = None
        hollow = TensorAwareStateDict.from_state_dict(fresh())
        hollow.pop_tensors()
        it, back = mgr.recover_state_dict([1], hollow=hollow)
    else:
        it, back = mgr.recover_state_dict([1])
    assert it == 9
    assert torch.equal(back["model"]["w"], ref["w"]) and torch.equal(back["optimizer"]["state"][1], ref["m"])
    assert set(back) == {"iteration", "model", "optimizer"}


def test_state_dict_form_of_the_in_memory_checkpoint():
    run_distributed(_state_dict_rank, 2)
