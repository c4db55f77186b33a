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


# ------------------------------------------------------------------ NCCL issue-order model of the p2p transfers
def _simulate(pp, v, nmb, one_way_channels, overlap):
    """Replays the executor's transfers under NCCL's rules: the point-to-point operations of one communicator run
    in issue order (one stream per communicator per rank), and a send and its receive complete together, only
    when each is at the head of its rank's queue for that communicator and the send's data is computed.
    Returns True when every rank finishes its plan."""
    from collections import defaultdict, deque
    from megatron_lm_b200.parallel.schedules import build_pipeline_plan
    plans = [build_pipeline_plan(nmb, pp, r, v) for r in range(pp)]

    def comm_key(kind, sender_stage):
        if one_way_channels:
            return (kind, sender_stage)
        return frozenset((sender_stage, (sender_stage + 1) % pp))       # one communicator per neighbour pair

    def first_virtual(r, c): return r == 0 and c == 0
    def last_virtual(r, c): return r == pp - 1 and c == v - 1

    # issue order per rank: [(op, comm key, message id, step index that must be computed first or None)]
    queues = [defaultdict(deque) for _ in range(pp)]
    recv_of_step = [dict() for _ in range(pp)]
    for r, plan in enumerate(plans):
        posted = set()

        def post(idx):
            if idx >= len(plan) or idx in posted:
                return
            posted.add(idx)
            st = plan[idx]
            if st.kind == "F" and not first_virtual(r, st.chunk):
                key, msg = comm_key("F", (r - 1) % pp), ("F", (r - 1) % pp, st.chunk if r else st.chunk - 1, st.microbatch)
            elif st.kind == "B" and not last_virtual(r, st.chunk):
                key, msg = comm_key("B", r), ("B", r, st.chunk, st.microbatch)
            else:
                return
            queues[r][key].append(("recv", msg, None))
            recv_of_step[r][idx] = msg
        post(0)
        for idx, st in enumerate(plan):
            if overlap:
                post(idx + 1)
            post(idx)
            if st.kind == "F" and not last_virtual(r, st.chunk):
                queues[r][comm_key("F", r)].append(("send", ("F", r, st.chunk, st.microbatch), idx))
            if st.kind == "B" and not first_virtual(r, st.chunk):
                # the gradient of chunk c's input belongs to the sender's chunk (c on the previous stage, c-1 on wrap)
                sender = (r - 1) % pp
                queues[r][comm_key("B", sender)].append(("send", ("B", sender, st.chunk if r else st.chunk - 1,
                                                                  st.microbatch), idx))
    done_step = [-1] * pp                       # last computed step per rank
    received = [set() for _ in range(pp)]
    progress = True
    while progress:
        progress = False
        for r in range(pp):                    # compute as far as the received inputs allow
            while done_step[r] + 1 < len(plans[r]):
                nxt = done_step[r] + 1
                need = recv_of_step[r].get(nxt)
                if need is not None and need not in received[r]:
                    break
                done_step[r] = nxt
                progress = True
        for r in range(pp):                    # complete matching heads
            for key, q in queues[r].items():
                if not q or q[0][0] != "send":
                    continue
                _, msg, dep = q[0]
                if dep > done_step[r]:
                    continue
                dst = (r + 1) % pp if msg[0] == "F" else (r - 1) % pp
                dq = queues[dst].get(key)
                if dq and dq[0][0] == "recv" and dq[0][1] == msg:
                    q.popleft(); dq.popleft()
                    received[dst].add(msg)
                    progress = True
    return all(done_step[r] == len(plans[r]) - 1 for r in range(pp)) and \
        all(not q for r in range(pp) for q in queues[r].values())


@pytest.mark.parametrize("pp,v,nmb", [(2, 1, 4), (2, 2, 8), (4, 1, 8), (4, 2, 8), (4, 3, 12), (8, 2, 16), (2, 2, 64)])
@pytest.mark.parametrize("overlap", [False, True])
def test_one_way_channels_cannot_deadlock_under_nccl_ordering(pp, v, nmb, overlap):
    assert _simulate(pp, v, nmb, one_way_channels=True, overlap=overlap)


def test_shared_pair_communicator_would_deadlock():
    # the reason for the channels: with one communicator per neighbour pair the same transfers block each other
    assert not _simulate(2, 1, 4, one_way_channels=False, overlap=False)
    assert not _simulate(2, 2, 8, one_way_channels=False, overlap=True)
