"""Measure the GPU erasure-coded checkpoint: ``torchrun --nproc-per-node N -m megatron_lm_b200.checkpoint.ec_bench``.

Reports, device-timed and as the max over ranks: snapshot time, encode time and aggregate encode GB/s
(state bytes of all ranks / encode time), host-tier copy time, and the recovery time after ``--lose`` ranks
drop their device state (decode launch on the lost ranks + roll-back copy on all).  The rebuilt bytes are
compared with the originals.  State is synthetic: ``--state-gb`` random bytes per rank (the Llama-7B run
with distributed optimizer holds about 13.5 GB per rank on 8 GPUs).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--state-gb", type=float, default=2.0)
    # long names: a launcher that parses abbreviations (torchrun -m ...) must not mistake them for its own flags
    ap.add_argument("--data-shards", "--k", dest="k", type=int, default=None)
    ap.add_argument("--parity-shards", "--m", dest="m", type=int, default=2)
    ap.add_argument("--chunk-mib", type=float, default=1.0)
    ap.add_argument("--lose", type=int, default=2)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--encode-blocks", type=int, default=0)
    ap.add_argument("--no-host-tier", action="store_true")
    ap.add_argument("--direct-loads", action="store_true",
                    help="parity kernel with plain peer loads instead of bulk copies staged through shared memory")
    a = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from .ec_gpu import GpuECCheckpoint
    nbytes = int(a.state_gb * 2 ** 30) // 16 * 16
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    state = torch.randint(0, 2 ** 31 - 1, (nbytes // 4,), dtype=torch.int32, device="cuda", generator=g)
    m = min(a.m, world - 1)
    k = a.k if a.k is not None else world - m
    mgr = GpuECCheckpoint(dist.group.WORLD, nbytes, k=k, m=m, chunk_bytes=int(a.chunk_mib * 2 ** 20),
                          host_tier=not a.no_host_tier, encode_blocks=a.encode_blocks, staged=not a.direct_loads)

    def mx(v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    enc, snap, host = [], [], []
    for it in range(a.iters):
        st = mgr.save([state], it)
        t0 = time.perf_counter()
        mgr.wait()
        host.append(mx((time.perf_counter() - t0) * 1e3))
        enc.append(mx(st["encode_ms"]))
        snap.append(mx(st["snapshot_ms"]))
    # lose ranks: the last `lose` ranks' device memory is wiped, then rebuilt from the peers
    lose = min(a.lose, m)
    lost = list(range(world - lose, world))
    ref = state.clone()
    if rank in lost:
        mgr.drop_device_state()
        state.zero_()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    mgr.recover(lost, [state])
    e1.record()
    torch.cuda.synchronize()
    rec_ms = mx(e0.elapsed_time(e1))
    ok = torch.tensor([int(torch.equal(state, ref))], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        total = nbytes * world
        best = min(enc[1:] or enc)
        print(json.dumps({"n_gpus": world, "k": k, "m": m, "chunk_mib": a.chunk_mib, "state_gb_per_rank": a.state_gb,
                          "snapshot_ms": min(snap), "encode_ms": best, "encode_GBps_aggregate": total / best / 1e6,
                          "nvlink_bytes_per_rank": nbytes * (k + m - 1) / k if world > 1 else 0,
                          "host_tier_ms": min(host), "lost_ranks": lost, "recovery_s": rec_ms / 1e3,
                          "byte_exact": bool(ok.item()), "stripes": len(mgr.plan.stripes),
                          "kernel": "direct peer loads" if a.direct_loads else "bulk copies staged through shared memory",
                          "encode_fraction_of_nvlink_roofline": (nbytes / 770e9) / (best / 1e3) if world > 1 else None}),
              flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
