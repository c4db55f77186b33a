"""Rank grid and group construction (no communication: virtual ranks)."""
import itertools

import pytest

from megatron_lm_b200.parallel import state
from megatron_lm_b200.parallel.state import RankGenerator


def test_default_order_groups_tp_fastest():
    g = RankGenerator(tp=2, ep=1, dp=2, pp=2, cp=1)
    assert g.get_ranks("tp") == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert g.get_ranks("dp") == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert g.get_ranks("pp") == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert g.get_ranks("tp-pp") == [[0, 1, 4, 5], [2, 3, 6, 7]]


def _oracle(sizes, order, token):
    """Independent enumeration: decode every rank into coordinates and bucket by the
    coordinates that are NOT in the token."""
    toks = order.split("-")
    dims = [sizes[t] for t in toks]
    world = 1
    for d in dims:
        world *= d
    sel = set(token.split("-"))
    buckets = {}
    for r in range(world):
        rem, coord = r, {}
        for t, d in zip(toks, dims):
            coord[t] = rem % d
            rem //= d
        key = tuple(coord[t] for t in reversed(toks) if t not in sel)
        inner = tuple(coord[t] for t in reversed(toks) if t in sel)
        buckets.setdefault(key, []).append((inner, r))
    return [[r for _, r in sorted(v)] for _, v in sorted(buckets.items())]


@pytest.mark.parametrize("order", ["tp-cp-ep-dp-pp", "tp-cp-ep-pp-dp", "tp-pp-dp-cp-ep"])
def test_rank_lists_match_independent_enumeration(order):
    for tp, cp, dp, pp in itertools.product([1, 2], [1, 2], [1, 3], [1, 2]):
        g = RankGenerator(tp=tp, ep=1, dp=dp, pp=pp, cp=cp, order=order)
        sizes = dict(tp=tp, cp=cp, ep=1, dp=dp, pp=pp)
        for token in ["tp", "pp", "dp", "cp", "dp-cp", "tp-pp", "tp-dp-cp", "tp-cp"]:
            assert g.get_ranks(token) == _oracle(sizes, order, token), (order, tp, cp, dp, pp, token)


def test_missing_dim_in_order_must_be_one():
    with pytest.raises(RuntimeError):
        RankGenerator(tp=2, ep=1, dp=1, pp=2, cp=1, order="tp-dp")
    g = RankGenerator(tp=2, ep=1, dp=2, pp=1, cp=1, order="tp-dp")
    assert g.world_size == 4


def test_virtual_initialize_sizes_and_ranks():
    state.fake_initialize_model_parallel(16, rank=13, tensor_model_parallel_size=2, pipeline_model_parallel_size=2,
                                         context_parallel_size=2)
    assert state.get_tensor_model_parallel_world_size() == 2
    assert state.get_pipeline_model_parallel_world_size() == 2
    assert state.get_context_parallel_world_size() == 2
    assert state.get_data_parallel_world_size() == 2
    assert state.get_data_parallel_world_size(with_context_parallel=True) == 4
    # rank 13 = tp 1, cp 0, dp 1, pp 1 with tp fastest: 1 + 2*0 + 4*1 + 8*1
    assert state.get_tensor_model_parallel_rank() == 1
    assert state.get_context_parallel_rank() == 0
    assert state.get_data_parallel_rank() == 1
    assert state.get_pipeline_model_parallel_rank() == 1
    assert state.is_pipeline_last_stage() and not state.is_pipeline_first_stage()
    assert state.get_pipeline_model_parallel_prev_rank() == 5
    assert state.get_group_ranks("embd") == [5, 13]
    assert state.is_rank_in_embedding_group()


def test_expert_grid_shares_pipeline_groups():
    state.fake_initialize_model_parallel(8, rank=5, tensor_model_parallel_size=2, expert_model_parallel_size=4,
                                         expert_tensor_parallel_size=1)
    assert state.get_expert_model_parallel_world_size() == 4
    assert state.get_expert_tensor_parallel_world_size() == 1
    assert state.get_expert_data_parallel_world_size() == 2
    assert state.get_group_ranks("ep") == [4, 5, 6, 7]
    assert state.get_group_ranks("edp") == [1, 5]


def test_bad_sizes_rejected():
    with pytest.raises(RuntimeError):
        state.fake_initialize_model_parallel(6, tensor_model_parallel_size=4)
    with pytest.raises(RuntimeError):
        state.fake_initialize_model_parallel(8, tensor_model_parallel_size=2, virtual_pipeline_model_parallel_size=2)


def test_virtual_pipeline_rank_affects_first_last():
    state.fake_initialize_model_parallel(4, rank=0, pipeline_model_parallel_size=4,
                                         virtual_pipeline_model_parallel_size=2)
    assert state.is_pipeline_first_stage(ignore_virtual=False)
    state.set_virtual_pipeline_model_parallel_rank(1)
    assert not state.is_pipeline_first_stage(ignore_virtual=False)
    assert state.is_pipeline_first_stage(ignore_virtual=True)


def test_hierarchical_cp_groups():
    state.fake_initialize_model_parallel(8, rank=3, context_parallel_size=8, hierarchical_context_parallel_sizes=[2, 4])
    assert state.get_group_ranks("hcp0") == [2, 3]
    assert state.get_group_ranks("hcp1") == [1, 3, 5, 7]
