#!/usr/bin/env python
"""Pre-train a LLaVA-style vision-language model on mock image + text data.

Reference: pretrain_vlm.py (model_provider :48, mock dataset provider :217, forward_step :363).
"""
import os
import sys
from copy import deepcopy
from functools import partial

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from megatron_lm_b200.models.multimodal import DEFAULT_IMAGE_TOKEN_INDEX, LLaVAModel  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    print_rank_0("building a multimodal model ...")
    vis = deepcopy(config)
    vis.num_layers = getattr(args, "encoder_num_layers", None) or config.num_layers
    vis.pipeline_model_parallel_size, vis.virtual_pipeline_model_parallel_size = 1, None
    vis.context_parallel_size = 1
    proj = deepcopy(config)
    proj.num_layers = 2
    model = LLaVAModel(config, args.padded_vocab_size, args.max_position_embeddings, vis, proj,
                       img_h=getattr(args, "img_h", 336), img_w=getattr(args, "img_w", 336),
                       patch_dim=getattr(args, "patch_dim", 14), pre_process=pre_process, post_process=post_process,
                       language_position_embedding_type=args.position_embedding_type,
                       drop_vision_class_token=getattr(args, "disable_vision_class_token", False),
                       share_embeddings_and_output_weights=not args.untie_embeddings_and_output_weights)
    if getattr(args, "freeze_LM", False) or getattr(args, "freeze_ViT", False):
        model.freeze(freeze_language_model=getattr(args, "freeze_LM", False),
                     freeze_vision_model=getattr(args, "freeze_ViT", False), freeze_vision_projection=False)
    return model


class MockMultimodalDataset(torch.utils.data.Dataset):
    def __init__(self, n, seq, vocab, img_h, img_w, seed=0):
        self.n, self.seq, self.vocab, self.hw, self.seed = n, seq, vocab, (img_h, img_w), seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed + i)
        toks = torch.randint(1, self.vocab, (self.seq + 1,), generator=g)
        toks[0] = DEFAULT_IMAGE_TOKEN_INDEX
        return {"image": torch.randn(3, *self.hw, generator=g), "tokens": toks[:-1], "labels": toks[1:],
                "loss_mask": torch.ones(self.seq), "position_ids": torch.arange(self.seq)}


def train_valid_test_datasets_provider(num_samples):
    args = get_args()
    mk = lambda n, s: MockMultimodalDataset(n, args.seq_length, args.padded_vocab_size, getattr(args, "img_h", 336),
                                            getattr(args, "img_w", 336), s) if n else None
    return mk(num_samples[0], 0), mk(num_samples[1], 1), mk(num_samples[2], 2)


def loss_func(loss_mask, output_tensor):
    losses = output_tensor.float().view(-1)
    mask = loss_mask.reshape(-1).float()
    total = torch.stack([torch.sum(losses * mask), mask.sum()])
    validate_loss(total[0], get_args())
    return total[0], total[1].to(torch.int64), {"lm loss": total.detach().clone()}


def forward_step(data_iterator, model):
    b = next(data_iterator)
    dev = torch.cuda.current_device() if torch.cuda.is_available() else "cpu"
    img, tok, lab, lm = (b[k].to(dev) for k in ("image", "tokens", "labels", "loss_mask"))
    dt = next(model.parameters()).dtype
    out, new_mask = model(img.to(dt), tok, labels=lab, loss_mask=lm)
    return out, partial(loss_func, new_mask)


def add_vlm_args(parser):
    """Flags of the vision-language program (reference: pretrain_vlm.py:384 ``add_vlm_extra_args``)."""
    g = parser.add_argument_group(title="vision language model")
    g.add_argument("--disable-vision-class-token", action="store_true",
                   help="drop the class token of the vision model before the projection")
    g.add_argument("--freeze-LM", action="store_true", dest="freeze_LM", help="train without updating the language model")
    g.add_argument("--freeze-ViT", action="store_true", dest="freeze_ViT", help="train without updating the vision model")
    return parser


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step, extra_args_provider=add_vlm_args,
             args_defaults={"tokenizer_type": "NullTokenizer"})
