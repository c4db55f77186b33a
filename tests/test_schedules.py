"""Pipeline plan generation: warm-up counts, virtual-microbatch order, F/B pairing (pure CPU)."""
import pytest

from megatron_lm_b200.parallel.schedules import (build_pipeline_plan, convert_schedule_table_to_order,
                                                 get_pp_rank_microbatches, get_schedule_table)


def test_schedule_table_worked_example():
    # PP2, 2 chunks, 5 microbatches, group size 3
    t = get_schedule_table(5, 2, 3)
    assert [m for m, _ in t] == [0, 1, 2, 0, 1, 2, 3, 4, 3, 4]
    assert [c for _, c in t] == [0, 0, 0, 1, 1, 1, 0, 0, 1, 1]


@pytest.mark.parametrize("pp,rank,v,nmb,g,expect", [
    (4, 0, 1, 8, 4, 3), (4, 3, 1, 8, 4, 0), (2, 0, 2, 8, 2, (2 - 0 - 1) * 2 + 1 * 2),
    (4, 1, 2, 16, 4, (4 - 1 - 1) * 2 + 1 * 4), (4, 0, 3, 4, 4, 12)])
def test_warmup_counts(pp, rank, v, nmb, g, expect):
    total, all_warm, warm, rem = get_pp_rank_microbatches(nmb, v, g, pp, rank)
    assert total == nmb * v
    assert warm == min(expect, total)
    assert rem == total - warm
    assert all_warm == (expect >= total)


def test_order_conversion_matches_plan():
    for pp, v, nmb, g in [(2, 2, 4, 2), (4, 2, 8, 4), (2, 3, 5, 3), (4, 4, 8, 4)]:
        for rank in range(pp):
            total, _, warm, _ = get_pp_rank_microbatches(nmb, v, g, pp, rank)
            table = get_schedule_table(nmb, v, g)
            order = convert_schedule_table_to_order(warm, v, table)
            plan = build_pipeline_plan(nmb, pp, rank, v, g)
            got = [(s.chunk + 1) if s.kind == "F" else -(s.chunk + 1) for s in plan]
            # order uses +c for forward of chunk c-1, and (c - v) for the backward of forward-chunk c,
            # i.e. -(v - c) which is minus (mirrored chunk + 1)
            assert got == order, (pp, v, nmb, g, rank)


@pytest.mark.parametrize("pp,v,nmb", [(2, 1, 4), (4, 1, 8), (2, 2, 4), (4, 2, 8), (4, 2, 12)])
def test_plan_is_a_valid_schedule(pp, v, nmb):
    for rank in range(pp):
        plan = build_pipeline_plan(nmb, pp, rank, v, pp)
        f = [(s.chunk, s.microbatch) for s in plan if s.kind == "F"]
        b = [(s.chunk, s.microbatch) for s in plan if s.kind == "B"]
        assert len(f) == len(b) == nmb * v
        assert sorted(f) == sorted(b) == sorted((c, m) for c in range(v) for m in range(nmb))
        seen = set()
        for s in plan:                     # a backward never precedes its forward
            if s.kind == "F":
                seen.add((s.chunk, s.microbatch))
            else:
                assert (s.chunk, s.microbatch) in seen
        for c in range(v):                 # per chunk, microbatches are processed in order
            assert [m for cc, m in f if cc == c] == list(range(nmb))
            assert [m for cc, m in b if cc == c] == list(range(nmb))


def test_cross_rank_dependencies_are_satisfiable():
    """Simulate all ranks step by step: every receive has a matching earlier send (no deadlock)."""
    for pp, v, nmb in [(2, 1, 3), (4, 1, 8), (2, 2, 4), (4, 2, 8)]:
        plans = [build_pipeline_plan(nmb, pp, r, v, pp) for r in range(pp)]
        pos = [0] * pp
        done = set()

        def ready(r, s):
            if s.kind == "F":
                if r == 0 and s.chunk == 0:
                    return True
                pr, pc = (r - 1, s.chunk) if r > 0 else (pp - 1, s.chunk - 1)
                return ("F", pr, pc, s.microbatch) in done
            if r == pp - 1 and s.chunk == v - 1:
                return ("F", r, s.chunk, s.microbatch) in done
            nr, nc = (r + 1, s.chunk) if r < pp - 1 else (0, s.chunk + 1)
            return ("B", nr, nc, s.microbatch) in done
        progress = True
        while progress:
            progress = False
            for r in range(pp):
                while pos[r] < len(plans[r]) and ready(r, plans[r][pos[r]]):
                    s = plans[r][pos[r]]
                    done.add((s.kind, r, s.chunk, s.microbatch))
                    pos[r] += 1
                    progress = True
        assert all(pos[r] == len(plans[r]) for r in range(pp)), (pp, v, nmb, pos)


def test_forward_only_plan():
    plan = build_pipeline_plan(4, 2, 0, 2, 2, forward_only=True)
    assert all(s.kind == "F" for s in plan) and len(plan) == 8
