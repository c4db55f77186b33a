#!/usr/bin/env python
"""Pre-train a GPT / Llama / Mixtral-style model.

Usage mirrors the reference entry script (pretrain_gpt.py:95 model_provider, :285 forward_step,
:223 loss_func, :357 datasets provider): the same flags, launched with torchrun, e.g.

    torchrun --nproc-per-node 8 pretrain_gpt.py --tensor-model-parallel-size 4 \
        --pipeline-model-parallel-size 2 --num-layers 32 --hidden-size 4096 ... --mock-data
"""
import os
import sys
from functools import partial

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from megatron_lm_b200.data.gpt_dataset import (BlendedMegatronDatasetBuilder, GPTDataset, GPTDatasetConfig,  # noqa: E402
                                               MockGPTDataset)
from megatron_lm_b200.models.gpt import GPTModel  # noqa: E402
from megatron_lm_b200.parallel import state  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.batch import get_batch_on_this_cp_rank, get_batch_on_this_tp_rank  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    print_rank_0("building GPT model ...")
    return GPTModel(config, vocab_size=args.padded_vocab_size, max_sequence_length=args.max_position_embeddings,
                    pre_process=pre_process, post_process=post_process, fp16_lm_cross_entropy=args.fp16_lm_cross_entropy,
                    parallel_output=True,
                    share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                    position_embedding_type=args.position_embedding_type, rotary_percent=args.rotary_percent,
                    rotary_base=args.rotary_base, rope_scaling=getattr(args, "use_rope_scaling", False),
                    rope_scaling_factor=getattr(args, "rope_scaling_factor", 8.0),
                    seq_len_interpolation_factor=args.rotary_seq_len_interpolation_factor, vp_stage=vp_stage)


def get_batch(data_iterator):
    if not (state.is_pipeline_first_stage() or state.is_pipeline_last_stage()):
        return None, None, None, None, None
    batch = get_batch_on_this_tp_rank(data_iterator, get_args())
    batch = get_batch_on_this_cp_rank(batch)
    return batch["tokens"], batch["labels"], batch["loss_mask"], batch.get("attention_mask"), batch["position_ids"]


def loss_func(loss_mask, output_tensor):
    losses = output_tensor.float().view(-1)
    mask = loss_mask.view(-1).float()
    total = torch.stack([torch.sum(losses * mask), mask.sum()])
    if state.get_context_parallel_world_size() > 1:
        torch.distributed.all_reduce(total, group=state.get_context_parallel_group())
    validate_loss(total[0], get_args())
    return total[0], total[1].to(torch.int64), {"lm loss": total.detach().clone()}


def forward_step(data_iterator, model):
    tokens, labels, loss_mask, attention_mask, position_ids = get_batch(data_iterator)
    out = model(tokens, position_ids, attention_mask, labels=labels)
    return out, partial(loss_func, loss_mask)


def train_valid_test_datasets_provider(num_samples):
    args = get_args()
    def as_blend(paths):
        if not paths:
            return None
        if len(paths) == 1:
            return ([paths[0]], None)
        return ([paths[i] for i in range(1, len(paths), 2)], [float(paths[i]) for i in range(0, len(paths), 2)])
    blend = as_blend(args.data_path)
    # --train-data-path / --valid-data-path / --test-data-path: one corpus (or blend) per split instead of one
    # corpus cut by --split
    per_split = [as_blend(getattr(args, k, None)) for k in ("train_data_path", "valid_data_path", "test_data_path")]
    per_split = per_split if any(b is not None for b in per_split) else None
    if per_split is not None:
        blend = None
    cfg = GPTDatasetConfig(random_seed=args.seed, sequence_length=args.seq_length, blend=blend,
                           blend_per_split=per_split, split=None if per_split is not None else args.split,
                           path_to_cache=args.data_cache_path, mmap_bin_files=args.mmap_bin_files, mock=args.mock_data,
                           tokenizer=args.tokenizer, reset_position_ids=args.reset_position_ids,
                           reset_attention_mask=args.reset_attention_mask, eod_mask_loss=args.eod_mask_loss,
                           create_attention_mask=args.create_attention_mask_in_dataloader)
    if getattr(args, "sft", False):
        # supervised fine-tuning: --data-path names a JSONL file of conversations; loss on the assistant turns only
        from megatron_lm_b200.data.sft_dataset import TEMPLATES, SFTDataset, default_chat_template
        template = TEMPLATES.get(getattr(args, "sft_tokenizer_prompt_format", None), default_chat_template)

        def make(n, seed):
            return SFTDataset(args.data_path[-1], args.tokenizer, args.seq_length, n, template=template,
                              seed=seed) if n else None
        print_rank_0("building train, validation and test datasets for supervised fine-tuning ...")
        return make(num_samples[0], args.seed), make(num_samples[1], args.seed + 1), make(num_samples[2], args.seed + 2)
    cls = MockGPTDataset if cfg.mock else GPTDataset
    print_rank_0("building train, validation and test datasets for GPT ...")
    return BlendedMegatronDatasetBuilder(cls, num_samples, lambda: True, cfg).build()


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step,
             args_defaults={"tokenizer_type": "GPT2BPETokenizer"})
