#!/usr/bin/env python
"""Headline benchmark: Llama-2-7B-style pre-training step, tokens/s (whole job).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 3 --warmup 3

Config (fixed): 32 layers, hidden 4096, 32 heads (MHA), SwiGLU FFN 11008, RMSNorm eps 1e-5,
RoPE theta 1e4, seq 4096, vocab 32000, micro-batch 1, global batch 64, bf16 compute with fp32
master weights / fp32 gradient accumulation, AdamW, grad clipping 1.0; synthetic uniform-random
tokens, random-init weights.  Parallel layout by GPU count: 1 -> tp1 pp1, 2 -> tp2, 4 -> tp4,
8 -> tp4 pp2 with 2 virtual stages; sequence parallel (with the fused all-gather->GEMM / GEMM->reduce-scatter
kernels, pipeline parallelism included) and the distributed optimizer are on whenever tp > 1 / dp > 1.  Total work is fixed as N grows (strong scaling).

One timed loop of K optimizer steps (after W warm-up steps) carries both clocks.  Every step copies its
[64, 4097] int64 token batch from pinned host memory, runs, and reads the step's loss back to the host:
  * device-timed: a pair of CUDA events around each step alone (copy and read-back outside), summed over the
    K steps, max over ranks -> ``value``;
  * end to end: wall clock of the whole loop, copies and read-backs included -> ``e2e``.
Both arms use the same loop.
``--impl reference`` runs the unmodified reference library (megatron.core from baseline/_ref)
on the same model/config through its own public API.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))

LLAMA7B = dict(num_layers=32, hidden_size=4096, num_attention_heads=32, ffn_hidden_size=11008, seq_length=4096,
               vocab_size=32000, micro_batch_size=1, global_batch_size=64)
GPT3_1P3B = dict(num_layers=24, hidden_size=2048, num_attention_heads=16, ffn_hidden_size=8192, seq_length=2048,
                 vocab_size=50304, micro_batch_size=4, global_batch_size=256)
MIXTRAL = dict(num_layers=16, hidden_size=4096, num_attention_heads=32, num_query_groups=8, ffn_hidden_size=14336,
               seq_length=4096, vocab_size=32000, micro_batch_size=1, global_batch_size=64, num_experts=8, topk=2)
MODELS = {"llama7b": LLAMA7B, "gpt3-1.3b": GPT3_1P3B, "mixtral": MIXTRAL}
BASELINE_TOKENS_PER_SEC_PER_GPU = None      # the reference publishes no B200 number


def layout_for(n: int, config: str = "llama7b"):
    """(tp, pp, virtual stages, ep) for ``n`` GPUs.  llama7b (the headline): tp up to 4, then pp 2 with two
    virtual stages; gpt3-1.3b: tp 2 and the rest data parallel; mixtral: expert parallel over all GPUs."""
    if config == "gpt3-1.3b":
        return (2 if n >= 2 else 1, 1, None, 1)
    if config == "mixtral":
        if n < 4:
            raise SystemExit("the mixtral config holds 22.5 B parameters: it needs at least 4 GPUs (expert parallel)")
        return (1, 1, None, n)
    return {1: (1, 1, None, 1), 2: (2, 1, None, 1), 4: (4, 1, None, 1), 8: (4, 2, 2, 1)}[n]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def max_over_ranks(x: float, device) -> float:
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync():
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize()


# ----------------------------------------------------------------------------- our implementation
def run_ours(args):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.ops import _lib
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.random import model_parallel_cuda_manual_seed
    from megatron_lm_b200.training.training import setup_model_and_optimizer, train_step

    rank, world, local = dist_env()
    assert world == args.gpus, f"launched with {world} ranks for --gpus {args.gpus}"
    # diagnosis aid: if a multi-GPU run is still going after this many seconds, every thread's Python stack goes
    # to stderr (stdout keeps the single JSON line); MLB_BENCH_STACK_DUMP_S overrides, 0 turns it off
    dump_s = int(os.environ.get("MLB_BENCH_STACK_DUMP_S", "420" if world > 1 else "0"))
    if dump_s > 0:
        import faulthandler
        faulthandler.dump_traceback_later(dump_s, exit=False)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        from datetime import timedelta
        # a stuck collective ends with an error after ten minutes instead of holding the GPUs for the default thirty
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(minutes=10))
    tp, pp, vpp, ep = layout_for(args.gpus, args.config)
    if args.layout:                                   # debug only: "tp,pp,vpp" (vpp 0 = none)
        tp, pp, vpp = (int(x) for x in args.layout.split(","))
        vpp = vpp or None
    state.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                                    virtual_pipeline_model_parallel_size=vpp, expert_model_parallel_size=ep,
                                    create_gloo_process_groups=False)
    model_parallel_cuda_manual_seed(1234 + 100 * state.get_pipeline_model_parallel_rank())
    M = dict(MODELS[args.config])
    if args.layers:
        M["num_layers"] = args.layers
    if args.seq:
        M["seq_length"] = args.seq
    if args.tiny:
        # same layer count, micro-batch count and code path, matrices small enough that the GPU is never the limit:
        # the step time is then the host's cost of issuing a step
        M.update(hidden_size=512, ffn_hidden_size=1408, num_attention_heads=8, vocab_size=4096, seq_length=512)
    dp = world // (tp * pp)
    common = dict(
        num_layers=M["num_layers"], hidden_size=M["hidden_size"], num_attention_heads=M["num_attention_heads"],
        ffn_hidden_size=M["ffn_hidden_size"], hidden_dropout=0.0,
        attention_dropout=0.0, bf16=True, params_dtype=torch.bfloat16, tensor_model_parallel_size=tp,
        pipeline_model_parallel_size=pp, virtual_pipeline_model_parallel_size=vpp, sequence_parallel=tp > 1,
        pipeline_dtype=torch.bfloat16, tp_comm_overlap=args.tp_comm_overlap and tp > 1, init_method_std=0.02,
        overlap_p2p_comm=pp > 1, fp8=args.fp8, fp8_recipe=(args.fp8_recipe if args.fp8 else "delayed"))
    if args.config == "gpt3-1.3b":
        cfg = TransformerConfig(normalization="LayerNorm", layernorm_epsilon=1e-5, gated_linear_unit=False,
                                activation_func="gelu", add_bias_linear=True, **common)
        model_kw = dict(position_embedding_type="learned_absolute", share_embeddings_and_output_weights=True)
    elif args.config == "mixtral":
        cfg = TransformerConfig(normalization="RMSNorm", layernorm_epsilon=1e-5, gated_linear_unit=True,
                                activation_func="silu", add_bias_linear=False, num_query_groups=M["num_query_groups"],
                                num_moe_experts=M["num_experts"], moe_router_topk=M["topk"],
                                moe_ffn_hidden_size=M["ffn_hidden_size"], moe_aux_loss_coeff=1e-2,
                                moe_router_load_balancing_type="aux_loss", moe_grouped_gemm=True,
                                moe_token_dispatcher_type="flex" if ep > 1 else "alltoall",
                                expert_model_parallel_size=ep, **common)
        model_kw = dict(position_embedding_type="rope", rotary_base=1000000.0,
                        share_embeddings_and_output_weights=False)
    else:
        cfg = TransformerConfig(normalization="RMSNorm", layernorm_epsilon=1e-5, gated_linear_unit=True,
                                activation_func="silu", add_bias_linear=False, **common)
        model_kw = dict(position_embedding_type="rope", rotary_base=10000.0, share_embeddings_and_output_weights=False)

    def provider(pre_process=True, post_process=True, vp_stage=None):
        return GPTModel(cfg, vocab_size=M["vocab_size"], max_sequence_length=M["seq_length"], pre_process=pre_process,
                        post_process=post_process, vp_stage=vp_stage, **model_kw)

    ocfg = OptimizerConfig(optimizer="adam", lr=3e-4, min_lr=3e-5, weight_decay=0.1, adam_beta1=0.9, adam_beta2=0.95,
                           adam_eps=1e-8, clip_grad=1.0, bf16=True, params_dtype=torch.bfloat16,
                           use_distributed_optimizer=dp > 1)
    dcfg = DistributedDataParallelConfig(grad_reduce_in_fp32=True, overlap_grad_reduce=dp > 1,
                                         use_distributed_optimizer=dp > 1,
                                         peer_memory_collectives=not args.no_peer_dist_opt)
    model, opt, sched = setup_model_and_optimizer(
        provider, cfg, ocfg, dcfg,
        scheduler_kwargs=dict(lr=3e-4, min_lr=3e-5, lr_decay_style="cosine", train_iters=1000,
                              global_batch_size=M["global_batch_size"], lr_warmup_iters=10, weight_decay=0.1))
    fused = None
    if cfg.tp_comm_overlap:
        from megatron_lm_b200.ops.tp_fused import attach_fused_tp, detach_fused_tp
        fused = attach_fused_tp(model, cfg, M["seq_length"], M["micro_batch_size"])

    S, B, GB = M["seq_length"], M["micro_batch_size"], M["global_batch_size"]
    nmb = GB // (B * dp)
    gen = torch.Generator().manual_seed(1234 + state.get_data_parallel_rank())
    n_batches = args.warmup + args.steps              # a fresh batch for every step of the run
    host_batches = [torch.randint(0, M["vocab_size"], (nmb * B, S + 1), generator=gen, dtype=torch.int64).pin_memory()
                    for _ in range(n_batches)]
    h2d_bytes = host_batches[0].numel() * host_batches[0].element_size()

    def make_iters(batch):
        def gen():
            for i in range(nmb):
                rows = batch[i * B:(i + 1) * B]
                yield rows[:, :-1], rows[:, 1:]
        return [gen() for _ in model] if len(model) > 1 else gen()

    def forward_step(data_iterator, m):
        tokens, labels = next(data_iterator)
        out = m(tokens, labels=labels)

        def loss_func(output):
            loss = output.float().mean()
            return loss, {"lm loss": loss.detach()}
        return out, loss_func

    def one_step(batch_dev):
        return train_step(forward_step, make_iters(batch_dev), model, opt, sched, cfg, num_microbatches=nmb,
                          seq_length=S, micro_batch_size=B, global_batch_size=GB)

    def any_rank_timed_out() -> bool:
        st = _lib.status_word().clone()
        if world > 1:
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        return int(st.item()) != 0

    note = None
    for w in range(args.warmup):
        losses, *_ = one_step(host_batches[w].to(dev))
        if w == 0 and fused is not None and any_rank_timed_out():
            # A bounded wait of a fused kernel ran out in the first step (the kernels then drain at once, so the
            # step is short and its numbers are void).  Carry on with NCCL collectives around the plain GEMMs and
            # say so in the result instead of timing garbage.
            torch.cuda.synchronize()
            _lib.status_word().zero_()
            detach_fused_tp(model)
            fused = None
            note = "fused tensor-parallel kernels timed out in warm-up; ran with NCCL collectives instead"
            if rank == 0:
                print(note, file=sys.stderr, flush=True)
            if world > 1:
                dist.barrier()
            one_step(host_batches[w].to(dev))
    _lib.check_status()
    # ---- one timed loop of K steps carries both clocks.  Every step copies its batch from pinned host memory,
    # runs, and reads the loss back on the host.  Device time of a step: a pair of CUDA events around the step
    # alone (copy and read-back outside); end-to-end time: wall clock of the whole loop.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    _lib.launch_count = 0
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    host_issue_s = 0.0
    barrier_sync()
    t0 = time.perf_counter()
    loss_val = 0.0
    for k in range(args.steps):
        b = host_batches[args.warmup + k].to(dev, non_blocking=True)
        ev[k][0].record()
        h0 = time.perf_counter()
        losses, *_ = one_step(b)
        host_issue_s += time.perf_counter() - h0       # time the host needed to issue the step (no sync inside)
        ev[k][1].record()
        if pp > 1:
            # only the last pipeline stage holds the loss: every rank receives it, then reads it on the host
            lt = losses["lm loss"].detach().float().reshape(1) if losses else torch.zeros(1, device=dev)
            dist.all_reduce(lt, op=dist.ReduceOp.MAX)
            loss_val = float(lt.item())
        elif losses:
            loss_val = float(losses["lm loss"].item())
        else:
            torch.cuda.current_stream().synchronize()
    barrier_sync()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, dev)
    dev_ms = max_over_ranks(sum(a.elapsed_time(b_) for a, b_ in ev), dev)
    host_ms = max_over_ranks(host_issue_s * 1e3, dev)
    launches = _lib.launch_count
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status()
    tokens_per_step = GB * S
    value = tokens_per_step * args.steps / (dev_ms / 1e3)
    e2e = tokens_per_step * args.steps / (e2e_ms / 1e3)
    if rank == 0:
        from megatron_lm_b200.training.flops import flops_from_config
        fl = flops_from_config(cfg, GB, S, M["vocab_size"])
        par = f"tp{tp}pp{pp}" + (f"vpp{vpp}" if vpp else "") + f"dp{dp}" + (f"ep{ep}" if ep > 1 else "") + \
            ("-sp" if tp > 1 else "")
        names = {"llama7b": ("Llama-7B", "llama2-7b (32L h4096 32 heads ffn11008 swiglu rmsnorm rope)"),
                 "gpt3-1.3b": ("GPT-3 1.3B", "gpt3-1.3b (24L h2048 16 heads ffn8192 gelu layernorm learned positions)"),
                 "mixtral": ("Mixtral-style 8-expert MoE", "mixtral-style (16L h4096 32q/8kv heads, 8 experts top-2 "
                             "ffn14336 swiglu rmsnorm rope 1e6, aux loss 1e-2, dropless)")}[args.config]
        out = {
            "metric": f"tokens/sec (whole job) {names[0]} pre-training step", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / args.gpus / BASELINE_TOKENS_PER_SEC_PER_GPU) if BASELINE_TOKENS_PER_SEC_PER_GPU else None,
            "dtype": (("mxfp8" if args.fp8_recipe == "mxfp8" else "fp8") if args.fp8 else "bf16"), "data": "synthetic uniform-random tokens, random-init weights", "impl": "ours",
            "tokens_per_sec_per_gpu": value / args.gpus,
            "model_tflops_per_gpu": fl / (dev_ms / args.steps / 1e3) / 1e12 / args.gpus,
            "config": {"model": names[1] if not (args.layers or args.seq or args.tiny)
                       else f"{args.config} with debug overrides layers={args.layers} seq={args.seq} tiny={args.tiny} "
                            "(not a bench value)",
                       "global_batch": GB, "seq_len": S, "micro_batch": B, "parallelism": par,
                       "l2_note": "inputs and weights (>13 GB) far exceed the 126 MB L2 every step"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "last_loss": loss_val},
            "gpu_launches": launches,
            "host_issue_ms_per_step": host_ms / args.steps,
            "tp_comm_overlap": fused is not None,
            "timing": "one loop of K steps: device time = sum of per-step CUDA-event intervals (max over ranks), "
                      "e2e = wall clock of the same loop incl. the pinned-host batch copy and the loss read",
        }
        if note:
            out["note"] = note
        print(json.dumps(out), flush=True)
    dist.barrier()
    state.destroy_model_parallel()
    dist.destroy_process_group()


# ----------------------------------------------------------------------------- reference arm
def run_reference(args):
    ref = os.path.join(ROOT, "baseline", "_ref")
    rank, world, local = dist_env()
    if not os.path.isdir(os.path.join(ref, "megatron", "core")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this box"}))
        return
    sys.path.insert(0, ROOT)
    from baseline.run_reference import run
    run(args, ref, LLAMA7B, layout_for, ClockSampler, max_over_ranks, barrier_sync)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="llama7b", choices=sorted(MODELS),
                    help="llama7b is the headline benchmark; the others are the secondary configurations")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (result is not a bench value)")
    ap.add_argument("--layout", default=None, help="debug only: override the parallel layout as tp,pp,vpp")
    ap.add_argument("--no-peer-dist-opt", action="store_true",
                    help="data-parallel layouts: distributed optimizer through NCCL instead of the peer-memory kernels")
    ap.add_argument("--tiny", action="store_true",
                    help="debug only: hidden 512 / seq 512 with the same layers and micro-batches - the step time is the "
                         "host's cost of issuing a step (result is not a bench value)")
    ap.add_argument("--seq", type=int, default=0,
                    help="debug only: override the sequence length; with a short one the step time is the host's cost of "
                         "issuing the step (result is not a bench value)")
    ap.add_argument("--tp-comm-overlap", action="store_true", default=True)
    ap.add_argument("--no-tp-comm-overlap", dest="tp_comm_overlap", action="store_false")
    ap.add_argument("--fp8", default=None, choices=["e4m3", "hybrid"],
                    help="FP8 variant: layer linears run FP8 GEMMs with per-tensor scales (reported as dtype fp8)")
    ap.add_argument("--fp8-recipe", default="tensorwise", choices=["tensorwise", "mxfp8"],
                    help="with --fp8: per-tensor current scaling, or block-scaled MXFP8 (1x32 blocks, E8M0 scales)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif os.environ.get("MLB_BENCH_PROFILE") and int(os.environ.get("RANK", "0")) == 0:
        # host-side profile of rank 0 (where the Python time of a step goes); the JSON line is then not a bench value
        import cProfile
        cProfile.runctx("run_ours(args)", globals(), {"args": args}, filename=os.environ["MLB_BENCH_PROFILE"])
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
