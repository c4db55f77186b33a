"""Reference arm of bench.py: the unmodified reference library (megatron.core installed under
baseline/_ref) training the same Llama-2-7B-style model through its own public API - GPTModel
with the library's local layer spec (Transformer Engine and Apex are not installed here, so its
fused/TE code path cannot be selected), DistributedDataParallel, get_megatron_optimizer and
get_forward_backward_func.  Nothing from megatron_lm_b200 is imported on this path.
"""
from __future__ import annotations

import json
import os
import sys
import time
import warnings


def run(args, ref_path, M, layout_for, ClockSampler, max_over_ranks, barrier_sync):
    warnings.filterwarnings("ignore")
    sys.path.insert(0, ref_path)
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    try:
        from megatron.core import parallel_state
        from megatron.core.distributed import DistributedDataParallel, DistributedDataParallelConfig, finalize_model_grads
        from megatron.core.models.gpt.gpt_layer_specs import get_gpt_layer_local_spec
        from megatron.core.models.gpt.gpt_model import GPTModel
        from megatron.core.optimizer import OptimizerConfig, get_megatron_optimizer
        from megatron.core.pipeline_parallel.schedules import get_forward_backward_func
        from megatron.core.tensor_parallel.random import model_parallel_cuda_manual_seed
        from megatron.core.transformer.module import Float16Module
        from megatron.core.transformer.transformer_config import TransformerConfig
    except Exception as e:   # pragma: no cover
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}))
        return

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29512")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    tp, pp, vpp = layout_for(args.gpus)[:3]
    if getattr(args, "layout", None):                 # debug only: "tp,pp,vpp" (vpp 0 = none)
        tp, pp, vpp = (int(x) for x in args.layout.split(","))
        vpp = vpp or None
    parallel_state.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                                             virtual_pipeline_model_parallel_size=vpp)
    model_parallel_cuda_manual_seed(1234)
    L = args.layers or M["num_layers"]
    dp = world // (tp * pp)
    try:
        cfg = TransformerConfig(
            num_layers=L, hidden_size=M["hidden_size"], num_attention_heads=M["num_attention_heads"],
            ffn_hidden_size=M["ffn_hidden_size"], normalization="RMSNorm", layernorm_epsilon=1e-5,
            gated_linear_unit=True, activation_func=torch.nn.functional.silu, add_bias_linear=False,
            hidden_dropout=0.0, attention_dropout=0.0, bf16=True, params_dtype=torch.bfloat16,
            pipeline_dtype=torch.bfloat16, tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
            virtual_pipeline_model_parallel_size=vpp, sequence_parallel=False, init_method_std=0.02,
            # sequence parallelism is off: the library's local layer spec builds torch norms, which assert
            # against it (it needs Transformer Engine or Apex norms, neither installable offline), so its
            # tensor-parallel runs use plain TP all-reduces - its own stock path for this spec
            # without a fused attention kernel the library keeps [b, np, s, s] scores per layer;
            # selective recompute of core attention is its own stock answer to that
            recompute_granularity="selective", gradient_accumulation_fusion=False, masked_softmax_fusion=False,
            bias_activation_fusion=False, bias_dropout_fusion=False, apply_rope_fusion=False,
            persist_layer_norm=False, attention_softmax_in_fp32=False)
        spec = get_gpt_layer_local_spec(normalization="RMSNorm")
        chunks = []
        vps = range(vpp) if (pp > 1 and vpp) else [None]
        for v in vps:
            if v is not None:
                parallel_state.set_virtual_pipeline_model_parallel_rank(v)
            # this library version wants the virtual stage named when it is asked about a chunk's position
            pre = parallel_state.is_pipeline_first_stage(ignore_virtual=False, vp_stage=v) if v is not None \
                else parallel_state.is_pipeline_first_stage()
            post = parallel_state.is_pipeline_last_stage(ignore_virtual=False, vp_stage=v) if v is not None \
                else parallel_state.is_pipeline_last_stage()
            kw = dict(vp_stage=v) if v is not None else {}
            m = GPTModel(config=cfg, transformer_layer_spec=spec, vocab_size=M["vocab_size"],
                         max_sequence_length=M["seq_length"], pre_process=pre, post_process=post,
                         position_embedding_type="rope", rotary_base=10000, share_embeddings_and_output_weights=False,
                         **kw)
            m.cuda(dev)
            chunks.append(Float16Module(cfg, m))
        if vpp:
            parallel_state.set_virtual_pipeline_model_parallel_rank(0)
        dcfg = DistributedDataParallelConfig(grad_reduce_in_fp32=True, overlap_grad_reduce=False,
                                             use_distributed_optimizer=dp > 1)
        model = [DistributedDataParallel(config=cfg, ddp_config=dcfg, module=c, disable_bucketing=(i > 0))
                 for i, c in enumerate(chunks)]
        ocfg = OptimizerConfig(optimizer="adam", lr=3e-4, min_lr=3e-5, weight_decay=0.1, adam_beta1=0.9,
                               adam_beta2=0.95, adam_eps=1e-8, clip_grad=1.0, bf16=True,
                               params_dtype=torch.bfloat16, use_distributed_optimizer=dp > 1)
        opt = get_megatron_optimizer(ocfg, model)
        cfg.finalize_model_grads_func = finalize_model_grads
        cfg.grad_scale_func = opt.scale_loss
        if len(model) == 1:
            cfg.no_sync_func = model[0].no_sync
        else:
            cfg.no_sync_func = [m.no_sync for m in model]
    except Exception as e:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"model setup failed: {type(e).__name__}: {e}"[:300]}))
        dist.destroy_process_group()
        return

    S, B, GB = M["seq_length"], M["micro_batch_size"], M["global_batch_size"]
    nmb = GB // (B * dp)
    gen = torch.Generator().manual_seed(1234 + parallel_state.get_data_parallel_rank())
    host_batches = [torch.randint(0, M["vocab_size"], (nmb * B, S + 1), generator=gen, dtype=torch.int64).pin_memory()
                    for _ in range(2)]
    h2d_bytes = host_batches[0].numel() * 8
    pos = torch.arange(S, device=dev).unsqueeze(0).expand(B, S).contiguous()
    fb = get_forward_backward_func()

    def make_iters(batch):
        def gen_():
            for i in range(nmb):
                rows = batch[i * B:(i + 1) * B]
                yield rows[:, :-1].contiguous(), rows[:, 1:].contiguous()
        return [gen_() for _ in model] if len(model) > 1 else gen_()

    def forward_step(it, m):
        tokens, labels = next(it)
        out = m(tokens, pos, None, labels=labels)

        def loss_func(output):
            loss = output.float().mean()
            return loss, {"lm loss": loss.detach()}
        return out, loss_func

    def one_step(batch):
        for m in model:
            m.zero_grad_buffer()
        opt.zero_grad()
        losses = fb(forward_step_func=forward_step, data_iterator=make_iters(batch),
                    model=model if len(model) > 1 else model[0], num_microbatches=nmb, seq_length=S,
                    micro_batch_size=B, forward_only=False)
        opt.step()
        return losses

    try:
        dev_batches = [b.to(dev) for b in host_batches]
        for w in range(args.warmup):
            one_step(dev_batches[w % 2])
        # One loop of K steps carries both clocks (the same structure as the other arm): every step copies its
        # batch from pinned host memory, runs, and reads the loss back; the device time of a step is a pair of
        # CUDA events around the step alone, the end-to-end time is the wall clock of the whole loop.
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        barrier_sync()
        t0 = time.perf_counter()
        loss_val = 0.0
        for k in range(args.steps):
            b = host_batches[k % 2].to(dev, non_blocking=True)
            ev[k][0].record()
            losses = one_step(b)
            ev[k][1].record()
            if pp > 1:
                lt = torch.stack([d["lm loss"] for d in losses]).mean().reshape(1) if losses else torch.zeros(1, device=dev)
                dist.all_reduce(lt, op=dist.ReduceOp.MAX)
                loss_val = float(lt.item())
            elif losses:
                loss_val = float(torch.stack([d["lm loss"] for d in losses]).mean().item())
            else:
                torch.cuda.current_stream().synchronize()
        barrier_sync()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, dev)
        dev_ms = max_over_ranks(sum(a.elapsed_time(b_) for a, b_ in ev), dev)
        clocks = sampler.stop() if rank == 0 else None
    except Exception as e:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"training step failed: {type(e).__name__}: {e}"[:300]}))
        return
    tokens_per_step = GB * S
    value = tokens_per_step * args.steps / (dev_ms / 1e3)
    e2e = tokens_per_step * args.steps / (e2e_ms / 1e3)
    if rank == 0:
        par = f"tp{tp}pp{pp}" + (f"vpp{vpp}" if vpp else "") + f"dp{dp}" + ("-nosp (the local layer spec has no sequence-parallel norm)" if tp > 1 else "")
        print(json.dumps({
            "metric": "tokens/sec (whole job) Llama-7B pre-training step", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random tokens, random-init weights", "impl": "reference",
            "tokens_per_sec_per_gpu": value / args.gpus,
            "config": {"model": "llama2-7b (32L h4096 32 heads ffn11008 swiglu rmsnorm rope)" if not args.layers
                       else f"llama2-7b truncated to {args.layers} layers (debug only)",
                       "global_batch": GB, "seq_len": S, "micro_batch": B, "parallelism": par,
                       "variant": "megatron.core 0.14.0rc6 local layer spec (no TE/Apex installed), selective "
                                  "recompute of core attention"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "last_loss": loss_val,
                    "loss_note": "this arm cycles two fixed batches, so its loss falls by memorisation; it is not "
                                 "comparable with the other arm's loss on fresh batches"},
            "timing": "one loop of K steps: device time = sum of per-step CUDA-event intervals (max over ranks), "
                      "e2e = wall clock of the same loop incl. the pinned-host batch copy and the loss read",
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()
