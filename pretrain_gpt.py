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


def _gpt(args, config, pre_process, post_process, vp_stage):
    return GPTModel(config, vocab_size=args.padded_vocab_size, max_sequence_length=args.max_position_embeddings,
                    pre_process=pre_process, post_process=post_process, fp16_lm_cross_entropy=args.fp16_lm_cross_entropy,
                    parallel_output=True,
                    share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                    position_embedding_type=args.position_embedding_type, rotary_percent=args.rotary_percent,
                    rotary_base=args.rotary_base, rope_scaling=getattr(args, "use_rope_scaling", False),
                    rope_scaling_factor=getattr(args, "rope_scaling_factor", 8.0),
                    seq_len_interpolation_factor=args.rotary_seq_len_interpolation_factor, vp_stage=vp_stage)


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    print_rank_0("building GPT model ...")
    if getattr(args, "export_qk_l2_norm", False):
        config.qk_l2_norm = True
    model = _gpt(args, config, pre_process, post_process, vp_stage)
    if getattr(args, "export_kd_teacher_load", None) or getattr(args, "export_kd_cfg", None):
        model = _with_teacher(args, config, model, pre_process, post_process, vp_stage)
    return model


def _with_teacher(args, config, student, pre_process, post_process, vp_stage):
    """Knowledge distillation (--export-kd-teacher-load / --export-kd-cfg): a frozen teacher of the architecture in
    ``<teacher checkpoint>/model_config.yaml`` (the student's when that file is absent) rides along with the student
    (reference: megatron/post_training/model_provider.py:36-117)."""
    import copy
    import yaml
    from megatron_lm_b200.post_training.distillation import DistillationModel, load_distillation_config
    from megatron_lm_b200.training import checkpointing
    if vp_stage not in (None, 0) or (args.virtual_pipeline_model_parallel_size or 1) > 1:
        raise NotImplementedError("distillation with interleaved pipeline stages")
    t_cfg, t_args = copy.copy(config), copy.copy(args)
    load = getattr(args, "export_kd_teacher_load", None)
    if load and os.path.isfile(os.path.join(load, "model_config.yaml")):
        with open(os.path.join(load, "model_config.yaml")) as f:
            over = yaml.safe_load(f) or {}
        for k, v in over.items():
            if hasattr(t_cfg, k):
                setattr(t_cfg, k, v)
            if hasattr(t_args, k):
                setattr(t_args, k, v)
        if "num_query_groups" not in over and "num_attention_heads" in over and not over.get("group_query_attention"):
            t_cfg.num_query_groups = t_cfg.num_attention_heads
        if "kv_channels" not in over:
            t_cfg.kv_channels = t_cfg.hidden_size // t_cfg.num_attention_heads
    teacher = _gpt(t_args, t_cfg, pre_process, post_process, vp_stage)
    if load:
        t_args.load, t_args.finetune, t_args.no_load_optim, t_args.no_load_rng = load, True, True, True
        checkpointing.load_checkpoint([teacher], None, None, t_args, load_dir=load)
        print_rank_0(f"distillation teacher loaded from {load}")
    offsets = (getattr(student.decoder, "layer_offset", 0), getattr(teacher.decoder, "layer_offset", 0))
    kd = load_distillation_config(getattr(args, "export_kd_cfg", None), config, t_cfg,
                                  tp_group=state.get_tensor_model_parallel_group()
                                  if state.get_tensor_model_parallel_world_size() > 1 else None,
                                  layer_offsets=offsets, last_stage=post_process)
    model = DistillationModel(student, teacher, kd)
    if state.get_pipeline_model_parallel_world_size() > 1:
        config.adjust_tensor_shapes_fn = model.adjust_tensor_shapes
    return model


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


def distill_loss_func(loss_mask, model, output_tensor):
    from megatron_lm_b200.post_training.distillation import distillation_loss_func
    tp_group = state.get_tensor_model_parallel_group() if state.get_tensor_model_parallel_world_size() > 1 else None
    total, tokens, report = distillation_loss_func(loss_mask, output_tensor, model, tp_group)
    validate_loss(report["lm loss"][0], get_args())
    return total, tokens, report


def forward_step(data_iterator, model):
    tokens, labels, loss_mask, attention_mask, position_ids = get_batch(data_iterator)
    out = model(tokens, position_ids, attention_mask, labels=labels)
    if _DISTILL[0] is None:
        from megatron_lm_b200.post_training.distillation import unwrap_distillation_model
        _DISTILL[0] = unwrap_distillation_model(model) is not None
    if _DISTILL[0]:
        return out, partial(distill_loss_func, loss_mask, model)
    return out, partial(loss_func, loss_mask)


_DISTILL = [None]


def extra_args(parser):
    from megatron_lm_b200.post_training.arguments import add_modelopt_args
    return add_modelopt_args(parser)


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
                           create_attention_mask=args.create_attention_mask_in_dataloader,
                           object_storage_cache_path=getattr(args, "object_storage_cache_path", None))
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
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step, extra_args_provider=extra_args,
             args_defaults={"tokenizer_type": "GPT2BPETokenizer"})
