"""Back-of-the-envelope memory model (reference: megatron/training/theoretical_memory_usage.py:11-287):
weights + optimizer bytes per parameter (18 without / 6 + 12/dp with the distributed optimizer, for
bf16 params with fp32 gradients) and activation bytes per layer for the selective-recompute case
(``s*b*h*(18 + 4*ffn/h) / tp`` plus embedding, final norm and logits on the edge stages)."""
from __future__ import annotations

NUM_BYTES_IN_MEGABYTE = 1024 * 1024


def compute_weight_and_optimizer_memory(args, verbose: bool = False) -> float:
    kv = args.kv_channels or args.hidden_size // args.num_attention_heads
    qp = kv * args.num_attention_heads
    ng = args.num_query_groups if getattr(args, "group_query_attention", False) else args.num_attention_heads
    gated = 1.5 if args.swiglu else 1.0
    experts = 1 if args.num_experts is None else args.num_experts
    h = args.hidden_size
    per_layer = 2 * h * h * ((1 + ng / args.num_attention_heads) * qp / h
                             + (args.ffn_hidden_size / h) * experts * gated + 2 / h)
    transformer = per_layer * args.num_layers + 2 * h
    embed = h * args.padded_vocab_size
    untied = getattr(args, "untie_embeddings_and_output_weights", False)
    total_emb = embed * (2 if untied else 1)
    pp, tp = args.pipeline_model_parallel_size, args.tensor_model_parallel_size
    most_loaded = transformer / pp + embed
    if untied and pp == 1:
        most_loaded += embed
    most_loaded /= tp
    dp = args.data_parallel_size
    bytes_per_param = 18 if not args.use_distributed_optimizer else 6 + 12 / dp
    if verbose:
        print(f"parameters: {(transformer + total_emb) / 1e9:.2f} B total, {most_loaded / 1e9:.3f} B on the most loaded shard")
    return most_loaded * bytes_per_param


def compute_activation_memory(args, num_microbatches: int, verbose: bool = False) -> float:
    s, b, h = args.seq_length, args.micro_batch_size, args.hidden_size
    tp, pp = args.tensor_model_parallel_size, args.pipeline_model_parallel_size
    per_layer = s * b * h * (18 + 4 * args.ffn_hidden_size / h)
    act = per_layer * args.num_layers
    act += 8 * s * b * pp                  # embedding dropout masks of in-flight microbatches
    act += s * b * h * pp                  # embedding outputs
    vpp = getattr(args, "virtual_pipeline_model_parallel_size", None)
    if vpp is not None:
        act *= 1 + (pp - 1) / (pp * vpp)
    if vpp is None and pp > 1 and num_microbatches is not None:
        act *= min(1, num_microbatches / pp)
    if pp == 1:
        act += s * b * h * 4 * (1 + args.padded_vocab_size / h)
    return act / tp


def report_theoretical_memory(args, num_microbatches=None, verbose: bool = False) -> dict:
    w = compute_weight_and_optimizer_memory(args, verbose) / NUM_BYTES_IN_MEGABYTE
    out = {"weight_and_optimizer_mb": w}
    if getattr(args, "sequence_parallel", False) and getattr(args, "recompute_granularity", None) == "selective":
        a = compute_activation_memory(args, num_microbatches, verbose) / NUM_BYTES_IN_MEGABYTE
        out.update(activation_mb=a, total_mb=w + a)
    print(f"Theoretical memory footprints: weight and optimizer={w:.2f} MB" +
          (f", activation={out['activation_mb']:.2f} MB, total={out['total_mb']:.2f} MB" if "total_mb" in out else ""))
    return out
