"""Spawn one NCCL rank per GPU on this host and run a function in each."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, errq):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"] = str(rank), str(world), str(rank)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        fn(rank, world, *args)
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_on_gpus(fn, world: int, *args, timeout: float = 180.0):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    # poll: as soon as one rank fails, the others (likely blocked in a collective) are stopped
    import time
    deadline = time.time() + timeout
    while time.time() < deadline:
        if all(not p.is_alive() for p in procs):
            break
        if any((not p.is_alive()) and p.exitcode != 0 for p in procs):
            time.sleep(2.0)
            break
        time.sleep(0.2)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    for p in alive:
        p.join(10)
        if p.is_alive():
            p.kill()
    msgs = []
    while not errq.empty():
        msgs.append(errq.get())
    if msgs or alive or any(p.exitcode != 0 for p in procs):
        raise AssertionError("multi-GPU run failed:\n" + "\n".join(f"[rank {r}] {m}" for r, m in msgs)
                             + (f"\n{len(alive)} ranks timed out" if alive else ""))
