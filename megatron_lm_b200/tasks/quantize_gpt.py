"""Calibrate and quantise a GPT checkpoint.

    python -m megatron_lm_b200.tasks.quantize_gpt --load <ckpt> --save <out> --export-quant-cfg fp8 \
        --num-layers ... --hidden-size ... --tokenizer-type NullTokenizer --vocab-size 32000 \
        --calib-size 64 --calib-batch-size 4 [--valid-data corpus.txt | --data-path prefix | --mock-data]

The model is built from the training flags and loaded, a calibration set is run through it with the quantisers
recording ranges, the perplexity on that set is printed before and after, and the quantised model (ranges, folded
smoothing scales, FP8 weights for the ``*_real_quant`` recipes) is saved in the per-rank ``torch`` format.
Tensor-parallel models run one process per rank (launched with torchrun); ranges are reduced over the group.

Reference: tasks/quantize/calibrate_gpt.py:110-239 (calibration loop over WikiText, ``mtq.quantize`` through the
external library, before / after results).
"""
from __future__ import annotations

import math
import os
from typing import Iterator, List, Optional

import torch

from ..post_training import ptq
from ..post_training.arguments import add_modelopt_args, unsupported_set


def add_calib_args(parser):
    add_modelopt_args(parser)
    g = parser.add_argument_group(title="calibration")
    g.add_argument("--task", default="WIKITEXT103", help="name printed with the results")
    g.add_argument("--valid-data", nargs="*", default=None, help="text file(s) to calibrate on (needs a tokenizer)")
    g.add_argument("--calib-size", type=int, default=512, help="number of sequences")
    g.add_argument("--calib-batch-size", type=int, default=4)
    g.add_argument("--calib-seq-length", type=int, default=None, help="defaults to --seq-length")
    g.add_argument("--awq-alpha", type=float, default=0.5, help="SmoothQuant migration strength")
    return parser


def calibration_batches(args, tokenizer=None) -> Iterator[torch.Tensor]:
    """Token batches [b, s + 1] from text files, an indexed dataset, or (mock data) a fixed-seed random stream."""
    seq = args.calib_seq_length or args.seq_length
    n, bs = args.calib_size, args.calib_batch_size
    vocab = args.padded_vocab_size or args.vocab_size
    if args.valid_data:
        if tokenizer is None:
            raise SystemExit("--valid-data needs a tokenizer (--tokenizer-type ...)")
        ids: List[int] = []
        for path in args.valid_data:
            with open(path) as f:
                ids.extend(tokenizer.tokenize(f.read()))
        rows = [ids[i:i + seq + 1] for i in range(0, len(ids) - seq - 1, seq)][:n]
        if not rows:
            raise SystemExit(f"{args.valid_data}: fewer than {seq + 1} tokens")
        data = torch.tensor(rows, dtype=torch.long)
    elif getattr(args, "data_path", None) and not getattr(args, "mock_data", False):
        from ..data.indexed_dataset import IndexedDataset
        ds = IndexedDataset(args.data_path[-1])
        flat, i = [], 0
        while sum(len(x) for x in flat) < n * (seq + 1) and i < len(ds):
            flat.append(torch.as_tensor(ds[i].astype("int64")))
            i += 1
        flat = torch.cat(flat)
        rows = flat[: (flat.numel() // (seq + 1)) * (seq + 1)].view(-1, seq + 1)[:n]
        data = rows
    else:
        g = torch.Generator().manual_seed(1234)
        data = torch.randint(0, vocab, (n, seq + 1), generator=g)
    for i in range(0, data.shape[0], bs):
        yield data[i:i + bs]


@torch.no_grad()
def perplexity(model, batches: List[torch.Tensor], device) -> float:
    """exp(mean token loss) of a (possibly vocabulary-parallel) GPT model over ``batches``."""
    total, count = 0.0, 0
    for b in batches:
        b = b.to(device)
        tokens, labels = b[:, :-1].contiguous(), b[:, 1:].contiguous()
        pos = torch.arange(tokens.shape[1], device=device).unsqueeze(0).expand_as(tokens)
        loss = model(tokens, pos, None, labels=labels)
        total += loss.float().sum().item()
        count += labels.numel()
    return math.exp(total / max(count, 1))


def forward_loop(batches: List[torch.Tensor], device):
    def run(model):
        for b in batches:
            b = b.to(device)
            tokens = b[:, :-1].contiguous()
            pos = torch.arange(tokens.shape[1], device=device).unsqueeze(0).expand_as(tokens)
            model(tokens, pos, None)
    return run


def main(argv=None, store=None):
    from ..training import checkpointing
    from ..training.arguments import core_transformer_config_from_args
    from ..training.pretrain import initialize_megatron, print_rank_0
    from ..models.gpt import GPTModel
    from ..parallel import state
    args = initialize_megatron(add_calib_args, args_defaults={"save_interval": 1}, argv=argv, store=store)
    if state.get_pipeline_model_parallel_world_size() > 1:
        raise SystemExit("calibration runs the whole model in one process group position: use pipeline size 1")
    for k in unsupported_set(args):
        print_rank_0(f"WARNING: --{k.replace('_', '-')} has no effect in this program")
    cfg = core_transformer_config_from_args(args)
    if getattr(args, "export_qk_l2_norm", False):
        cfg.qk_l2_norm = True
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and args.distributed_backend == "nccl" \
        else torch.device("cpu")
    if dev.type == "cpu":
        cfg.use_cpu_initialization = True
    model = GPTModel(cfg, vocab_size=args.padded_vocab_size, max_sequence_length=args.max_position_embeddings,
                     parallel_output=True,
                     share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                     position_embedding_type=args.position_embedding_type, rotary_percent=args.rotary_percent,
                     rotary_base=args.rotary_base).to(dev)
    if args.load is not None:
        checkpointing.load_checkpoint([model], None, None, args, strict=False)
    model.eval()
    batches = list(calibration_batches(args, args.tokenizer))
    before = perplexity(model, batches, dev)
    fmt = args.export_quant_cfg
    if fmt in (None, "None"):
        fmt = args.export_real_quant_cfg
    if fmt in (None, "None"):
        raise SystemExit("give --export-quant-cfg (or --export-real-quant-cfg)")
    if args.export_real_quant_cfg not in (None, "None") and fmt in ("fp8", "fp8_blockwise"):
        fmt = fmt + "_real_quant"
    names = ptq.quantize(model, fmt, forward_loop(batches, dev), alpha=args.awq_alpha)
    after = perplexity(model, batches, dev)
    print_rank_0(f" {args.task}: {len(names)} linears quantised with {fmt}; perplexity on the calibration set "
                 f"{before:.4f} -> {after:.4f} ({len(batches)} batches)")
    if args.save is not None:
        args.ckpt_format = "torch"
        checkpointing.save_checkpoint(1, [model], None, None, args)
        print_rank_0(f" saved the quantised model to {os.path.abspath(args.save)}")
    return {"before": before, "after": after, "linears": len(names), "format": fmt}


if __name__ == "__main__":
    main()
