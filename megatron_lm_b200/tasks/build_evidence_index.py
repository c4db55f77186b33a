"""Embed an evidence file with a trained biencoder's context tower and save the embeddings for retrieval.

    torchrun --nproc-per-node 8 -m megatron_lm_b200.tasks.build_evidence_index \\
        --ict-load <biencoder checkpoint> --evidence-data-path wiki.tsv --embedding-path wiki_embeds.pt \\
        --indexer-batch-size 128 --retriever-seq-length 256 <model and tokenizer flags>

Reference: tools/create_doc_index.py / megatron/legacy/indexer.py:18 (``IndexBuilder``); flags of the biencoder
group (``--evidence-data-path``, ``--embedding-path``, ``--indexer-batch-size``, ``--indexer-log-interval``,
``--sample-rate``).
"""
from __future__ import annotations

import torch


def main(argv=None, store=None):
    from ..data.retrieval_index import IndexBuilder, OpenRetrievalEvidenceDataset
    from ..models.bert import BiEncoderModel
    from ..parallel import state
    from ..training import checkpointing
    from ..training.arguments import core_transformer_config_from_args
    from ..training.pretrain import argparse_namespace_copy, initialize_megatron, print_rank_0
    args = initialize_megatron(None, args_defaults={"tokenizer_type": "BertWordPieceLowerCase"}, argv=argv, store=store)
    if args.evidence_data_path is None or args.embedding_path is None:
        raise SystemExit("give --evidence-data-path and --embedding-path")
    if args.load is not None and args.ict_load is not None:
        raise SystemExit("give one of --load and --ict-load")
    if state.get_pipeline_model_parallel_world_size() > 1:
        raise SystemExit("the indexer runs the towers without pipeline parallelism")
    cfg = core_transformer_config_from_args(args)
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and args.distributed_backend == "nccl" \
        else torch.device("cpu")
    if dev.type == "cpu":
        cfg.use_cpu_initialization = True
    model = BiEncoderModel(cfg, args.padded_vocab_size, args.max_position_embeddings,
                           projection_dim=args.biencoder_projection_dim or (args.ict_head_size or 0),
                           shared_query_context_model=args.biencoder_shared_query_context_model).to(dev)
    load_dir = args.ict_load or args.load
    if load_dir is not None:
        ft = argparse_namespace_copy(args, finetune=True, no_load_optim=True, no_load_rng=True)
        checkpointing.load_checkpoint([model], None, None, ft, load_dir=load_dir, strict=False)
        print_rank_0(f"biencoder loaded from {load_dir}")
    seq = args.retriever_seq_length or args.seq_length
    dataset = OpenRetrievalEvidenceDataset(args.evidence_data_path, args.tokenizer, seq, sample_rate=args.sample_rate,
                                           seed=args.seed)
    print_rank_0(f" > evidence: {len(dataset)} rows from {args.evidence_data_path}")
    dp = state.get_data_parallel_world_size()
    builder = IndexBuilder(model, dataset, args.embedding_path, batch_size=args.indexer_batch_size,
                           log_interval=args.indexer_log_interval, dp_rank=state.get_data_parallel_rank(), dp_size=dp,
                           group=state.get_data_parallel_group() if dp > 1 else None, device=dev, log=print_rank_0)
    total = builder.build_and_save_index()
    print_rank_0(f" > saved {total} embeddings to {args.embedding_path}")
    return total


if __name__ == "__main__":
    main()
