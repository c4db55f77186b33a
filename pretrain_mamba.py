#!/usr/bin/env python
"""Pre-train a Mamba-2 or hybrid (state-space + attention + MLP) language model.

Same flags as ``pretrain_gpt.py`` plus ``--hybrid-attention-ratio``, ``--hybrid-mlp-ratio``,
``--hybrid-override-pattern``, ``--mamba-state-dim``, ``--mamba-head-dim``, ``--mamba-num-groups``
(reference: pretrain_mamba.py:52 model_provider, :193 forward_step).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from pretrain_gpt import forward_step, train_valid_test_datasets_provider  # noqa: E402
from megatron_lm_b200.models.mamba import MambaModel  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    print_rank_0("building Mamba model ...")
    return MambaModel(config, vocab_size=args.padded_vocab_size, max_sequence_length=args.max_position_embeddings,
                      pre_process=pre_process, post_process=post_process,
                      hybrid_attention_ratio=getattr(args, "hybrid_attention_ratio", 0.0),
                      hybrid_mlp_ratio=getattr(args, "hybrid_mlp_ratio", 0.0),
                      hybrid_override_pattern=getattr(args, "hybrid_override_pattern", None),
                      fp16_lm_cross_entropy=args.fp16_lm_cross_entropy, parallel_output=True,
                      share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights,
                      position_embedding_type=args.position_embedding_type, rotary_percent=args.rotary_percent,
                      rotary_base=args.rotary_base, d_state=getattr(args, "mamba_state_dim", 128),
                      headdim=getattr(args, "mamba_head_dim", 64), ngroups=getattr(args, "mamba_num_groups", 8))


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step,
             args_defaults={"tokenizer_type": "GPT2BPETokenizer"})
