"""Text-generation server program: builds a GPT model from the training command-line flags, loads a checkpoint and
serves ``PUT /api`` (the request / response format of the reference's server).

    python -m megatron_lm_b200.inference.run_server --load <dir> --num-layers ... --tokenizer-type ... --port 5000

Single GPU (or CPU) serving; tensor-parallel serving would run one such process per rank behind rank 0's HTTP
front end.  ``--server-model-type mamba`` serves pure and hybrid state-space models.
Reference: tools/run_text_generation_server.py, tools/run_mamba_text_generation_server.py (model + checkpoint +
``MegatronServer.run``).
"""
from __future__ import annotations

import torch

from ..models.gpt import GPTModel
from ..training import arguments as A
from .engine import DynamicInferenceEngine, StaticInferenceEngine
from .server import MegatronServer


def add_server_args(parser):
    g = parser.add_argument_group(title="text generation server")
    g.add_argument("--port", type=int, default=5000)
    g.add_argument("--host", default="0.0.0.0")
    g.add_argument("--engine", default="static", choices=["static", "dynamic"])
    g.add_argument("--server-model-type", default="gpt", choices=["gpt", "mamba"],
                   help="mamba: pure or hybrid state-space model (--hybrid-override-pattern ...), static engine")
    g.add_argument("--max-batch-size", type=int, default=None, help="defaults to --inference-max-requests")
    g.add_argument("--server-max-sequence-length", type=int, default=None)
    return parser


def build_engine(args, tokenizer=None):
    cfg = A.core_transformer_config_from_args(args)
    if not torch.cuda.is_available():
        cfg.use_cpu_initialization = True
    vocab = args.padded_vocab_size or getattr(args, "vocab_size", None)
    if vocab is None:
        raise SystemExit("the vocabulary size is unknown: give --vocab-size or a tokenizer")
    if getattr(args, "server_model_type", "gpt") == "mamba":
        # reference: tools/run_mamba_text_generation_server.py
        from ..models.mamba import MambaModel
        if args.engine == "dynamic" or getattr(args, "inference_dynamic_batching", False):
            raise SystemExit("state-space models are served by the static engine")
        model = MambaModel(cfg, vocab_size=vocab, max_sequence_length=args.max_position_embeddings, parallel_output=False,
                           hybrid_attention_ratio=getattr(args, "hybrid_attention_ratio", 0.0),
                           hybrid_mlp_ratio=getattr(args, "hybrid_mlp_ratio", 0.0),
                           hybrid_override_pattern=getattr(args, "hybrid_override_pattern", None),
                           share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                           position_embedding_type=args.position_embedding_type, rotary_percent=args.rotary_percent,
                           rotary_base=args.rotary_base, d_state=getattr(args, "mamba_state_dim", 128),
                           headdim=getattr(args, "mamba_head_dim", 64), ngroups=getattr(args, "mamba_num_groups", 8))
    else:
        model = GPTModel(cfg, vocab_size=vocab, max_sequence_length=args.max_position_embeddings, parallel_output=False,
                         share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                         position_embedding_type=args.position_embedding_type, rotary_percent=args.rotary_percent,
                         rotary_base=args.rotary_base)
    if torch.cuda.is_available():
        model = model.cuda()
    if args.load is not None:
        from ..training import checkpointing
        checkpointing.load_checkpoint([model], None, None, args, strict=False)
    model.eval()
    # the reference's inference flags size the engines: --inference-max-requests, --inference-max-seq-length,
    # --inference-dynamic-batching and its buffer settings
    if args.max_batch_size is None:
        args.max_batch_size = getattr(args, "inference_max_batch_size", 8)
    max_len = args.server_max_sequence_length or min(getattr(args, "inference_max_seq_length", 1 << 30),
                                                     args.max_position_embeddings)
    if args.engine == "dynamic" or getattr(args, "inference_dynamic_batching", False):
        return DynamicInferenceEngine(
            model, tokenizer=tokenizer, max_requests=args.max_batch_size, max_sequence_length=max_len,
            chunk_size=getattr(args, "inference_dynamic_batching_chunk_size", 256),
            buffer_size_gb=getattr(args, "inference_dynamic_batching_buffer_size_gb", None)
            if torch.cuda.is_available() else None,
            buffer_guaranteed_fraction=getattr(args, "inference_dynamic_batching_buffer_guaranteed_fraction", 0.0) or 0.0,
            buffer_overflow_factor=getattr(args, "inference_dynamic_batching_buffer_overflow_factor", None),
            max_requests_override=getattr(args, "inference_dynamic_batching_max_requests_override", None),
            max_tokens_override=getattr(args, "inference_dynamic_batching_max_tokens_override", None))
    return StaticInferenceEngine(model, tokenizer=tokenizer, max_batch_size=args.max_batch_size,
                                 max_sequence_length=max_len)


def main(argv=None, serve: bool = True, tokenizer=None):
    args = A.parse_args(add_server_args, argv=argv)
    if args.micro_batch_size is None:
        args.micro_batch_size = 1
    args = A.validate_args(args)
    if tokenizer is None and getattr(args, "tokenizer_type", None):
        from ..data.tokenizer import build_tokenizer
        tokenizer = build_tokenizer(args)
        if args.padded_vocab_size is None:
            args.padded_vocab_size = getattr(tokenizer, "vocab_size", None)
    server = MegatronServer(build_engine(args, tokenizer), max_batch=args.max_batch_size,
                            max_tokens_to_oom=getattr(args, "max_tokens_to_oom", None))
    if serve:
        print(f" > serving on {args.host}:{args.port}", flush=True)
        server.run(args.host, args.port)
    return server


if __name__ == "__main__":
    main()
