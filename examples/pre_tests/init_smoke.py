"""Bare process-group smoke test: every rank joins, all-reduces its rank and prints the sum.

    torchrun --nnodes N --node-rank R --nproc-per-node G --master-addr ADDR --master-port PORT \\
        examples/pre_tests/init_smoke.py
"""
import os

import torch
import torch.distributed as dist


def main():
    backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    t = torch.tensor([float(dist.get_rank())], device=dev)
    dist.all_reduce(t)
    n = dist.get_world_size()
    assert float(t) == n * (n - 1) / 2
    if dist.get_rank() == 0:
        print(f"{n} ranks joined over {backend}; all-reduce ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
