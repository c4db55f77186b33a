"""Stripe placement for the erasure-coded in-memory checkpoint ("parity-owner assignment").

Every rank contributes ``chunks_per_rank`` equal-size chunks of its flat state bytes.  A stripe has
k data chunks from k *different* ranks and m parity chunks whose owners are m *other* ranks, so
losing any m ranks loses at most m members of any stripe.  Rows rotate RAID-style: in row t the
parity owners are ranks (t*m + i) mod n; the remaining n - m ranks each contribute their next
unplaced chunk.  That requires k == n - m; a smaller k splits a row's data ranks into groups of k
that share the row's parity owners with separate parity slots.  When there are no spare ranks
(k == n), parity lives only in pinned host memory and is replicated on every member's host, so
any single GPU/process loss is still recoverable.  Parity chunks may additionally be mirrored to
the owner's host DRAM (second tier).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple


@dataclass
class Stripe:
    index: int
    data: List[Tuple[int, int]]           # (rank, chunk index on that rank)
    parity_owners: List[int]              # rank owning parity i (GPU tier), or all members for host-only
    host_only: bool = False


@dataclass
class StripePlan:
    n_ranks: int
    k: int
    m: int
    chunks_per_rank: int
    stripes: List[Stripe] = field(default_factory=list)

    def stripes_of_owner(self, rank: int) -> List[Tuple[int, int]]:
        """(stripe index, parity index) pairs whose parity this rank stores."""
        out = []
        for s in self.stripes:
            for i, o in enumerate(s.parity_owners):
                if o == rank or s.host_only:
                    out.append((s.index, i))
        return out

    def parity_chunks_per_rank(self) -> Dict[int, int]:
        c = {r: 0 for r in range(self.n_ranks)}
        for s in self.stripes:
            owners = range(self.n_ranks) if s.host_only else s.parity_owners
            for o in (set(r for r, _ in s.data) if s.host_only else owners):
                c[o] += self.m if s.host_only else 1
        return c

    def validate(self) -> None:
        seen = set()
        for s in self.stripes:
            ranks = [r for r, _ in s.data]
            assert len(set(ranks)) == len(ranks), "two chunks of one rank in a stripe"
            if not s.host_only:
                assert not (set(ranks) & set(s.parity_owners)), "parity co-located with stripe data"
                assert len(set(s.parity_owners)) == self.m
            for rc in s.data:
                assert rc not in seen
                seen.add(rc)
        assert len(seen) == self.n_ranks * self.chunks_per_rank, "some chunk is unprotected"


def plan_stripes(n_ranks: int, k: int, m: int, chunks_per_rank: int) -> StripePlan:
    if k < 1 or m < 1 or k > n_ranks:
        raise ValueError("need 1 <= k <= n_ranks and m >= 1")
    plan = StripePlan(n_ranks, k, m, chunks_per_rank)
    if k + m > n_ranks:
        if k != n_ranks:
            raise ValueError("k + m > n_ranks is only supported with k == n_ranks (host-tier parity)")
        for c in range(chunks_per_rank):
            plan.stripes.append(Stripe(c, [(r, c) for r in range(n_ranks)], list(range(n_ranks)), host_only=True))
        plan.validate()
        return plan
    nxt = [0] * n_ranks                                # next unplaced chunk of each rank
    t = 0
    while any(c < chunks_per_rank for c in nxt):
        owners = [(t * m + i) % n_ranks for i in range(m)]
        cand = [r for r in range(n_ranks) if r not in owners and nxt[r] < chunks_per_rank]
        # take data ranks in groups of k, most-behind ranks first so that everyone finishes together
        cand.sort(key=lambda r: (nxt[r], (r - t) % n_ranks))
        groups = [cand[i:i + k] for i in range(0, len(cand), k)]
        for gi, g in enumerate(groups):
            if len(g) < k and t < 4 * n_ranks * (chunks_per_rank + 1):
                # a short group waits for a later row unless only leftovers remain
                remaining = sum(chunks_per_rank - c for c in nxt)
                if remaining > len(g):
                    continue
            plan.stripes.append(Stripe(len(plan.stripes), [(r, nxt[r]) for r in g], owners))
            for r in g:
                nxt[r] += 1
        t += 1
        if t > 64 * n_ranks * (chunks_per_rank + 1):
            raise RuntimeError("stripe planning did not converge")
    plan.validate()
    return plan
