"""``python -m megatron_lm_b200.training.report_memory <training flags>``: print the analytic weight / optimizer /
activation memory estimate for a configuration without building the model
(reference: tools/report_theoretical_memory.py, megatron/training/theoretical_memory_usage.py:287)."""
from __future__ import annotations


def main(argv=None):
    from .arguments import parse_args, validate_args
    from .theoretical_memory_usage import report_theoretical_memory
    args = parse_args(argv=argv, ignore_unknown_args=True)
    mp = args.tensor_model_parallel_size * args.pipeline_model_parallel_size * max(getattr(args, "context_parallel_size", 1), 1)
    args.world_size = max(getattr(args, "world_size", None) or 1, mp)
    args.rank = 0
    try:
        args = validate_args(args)
    except Exception as e:                      # the estimate only needs the shape flags
        print(f"[report_memory] continuing without full validation: {e}")
    if getattr(args, "ffn_hidden_size", None) is None:
        args.ffn_hidden_size = 4 * args.hidden_size
    if getattr(args, "kv_channels", None) is None:
        args.kv_channels = args.hidden_size // args.num_attention_heads
    if getattr(args, "data_parallel_size", None) is None:
        mp = args.tensor_model_parallel_size * args.pipeline_model_parallel_size * max(getattr(args, "context_parallel_size", 1), 1)
        args.data_parallel_size = max(args.world_size // mp, 1)
    if getattr(args, "padded_vocab_size", None) is None:
        args.padded_vocab_size = getattr(args, "vocab_size", None) or 32000
    report_theoretical_memory(args, verbose=True)


if __name__ == "__main__":
    main()
