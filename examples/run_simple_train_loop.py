#!/usr/bin/env python
"""Minimal training loop on the library API only (no argument parser, no global state):

    torchrun --nproc-per-node 2 examples/run_simple_train_loop.py

initialise model parallelism (TP = world size), build a small GPT, wrap it in the data-parallel buffers,
build the optimizer, train a few steps on mock data with the pipeline-schedule entry point, save a
sharded checkpoint and load it back (reference counterpart: examples/run_simple_mcore_train_loop.py).
"""
import os
import sys
import tempfile
from functools import partial

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from megatron_lm_b200.checkpoint import sharded as ds  # noqa: E402
from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig  # noqa: E402
from megatron_lm_b200.models.gpt import GPTModel  # noqa: E402
from megatron_lm_b200.parallel import state  # noqa: E402
from megatron_lm_b200.parallel.random import model_parallel_cuda_manual_seed  # noqa: E402
from megatron_lm_b200.parallel.schedules import get_forward_backward_func  # noqa: E402
from megatron_lm_b200.training.training import setup_model_and_optimizer  # noqa: E402

SEQ, VOCAB, MBS = 64, 128, 2


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    state.initialize_model_parallel(tensor_model_parallel_size=world)
    model_parallel_cuda_manual_seed(123)
    dtype = torch.bfloat16 if cuda else torch.float32
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128,
                            tensor_model_parallel_size=world, sequence_parallel=world > 1, params_dtype=dtype,
                            bf16=cuda, use_cpu_initialization=not cuda, hidden_dropout=0.0, attention_dropout=0.0)
    provider = lambda pre_process, post_process, vp_stage=None: GPTModel(cfg, VOCAB, SEQ, pre_process, post_process)
    ocfg = OptimizerConfig(optimizer="adam", lr=1e-3, bf16=cuda, params_dtype=dtype, use_distributed_optimizer=False)
    model, optimizer, _ = setup_model_and_optimizer(provider, cfg, ocfg, DistributedDataParallelConfig())
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    g = torch.Generator().manual_seed(0)

    def batches():
        while True:
            t = torch.randint(0, VOCAB, (MBS, SEQ + 1), generator=g)
            yield {"tokens": t[:, :-1].to(dev), "labels": t[:, 1:].to(dev), "loss_mask": torch.ones(MBS, SEQ, device=dev)}

    def loss_func(mask, out):
        loss = (out.float() * mask).sum() / mask.sum()
        return loss, {"lm loss": loss.detach()}

    def forward_step(it, m):
        b = next(it)
        return m(b["tokens"], labels=b["labels"]), partial(loss_func, b["loss_mask"])

    fb = get_forward_backward_func()
    it = batches()
    for step in range(5):
        for m in model:
            m.zero_grad_buffer()
        optimizer.zero_grad()
        losses = fb(forward_step_func=forward_step, data_iterator=it, model=model, num_microbatches=2, seq_length=SEQ,
                    micro_batch_size=MBS, forward_only=False)
        optimizer.step()
        if rank == 0:
            print(f"step {step}: loss {float(losses[0]['lm loss']):.4f}", flush=True)
    ckpt = tempfile.mkdtemp() if rank == 0 else None
    box = [ckpt]
    dist.broadcast_object_list(box, src=0)
    sd = ds.model_sharded_state_dict(model[0].module, tp_rank=state.get_tensor_model_parallel_rank(), tp_size=world)
    ds.save(sd, box[0])
    loaded = ds.load(ds.model_sharded_state_dict(model[0].module, tp_rank=state.get_tensor_model_parallel_rank(),
                                                 tp_size=world), box[0])
    ds.load_model_from_sharded(model[0].module, loaded)
    if rank == 0:
        print("checkpoint saved and loaded from", box[0])
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
