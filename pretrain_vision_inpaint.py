#!/usr/bin/env python
"""Pre-train a vision transformer by in-painting: part of every image is hidden, the model reconstructs it.

Reference: pretrain_vision_inpaint.py (model provider :20, get_batch with the mask :33, loss = error on the hidden
region plus PSNR / SSIM of the reconstruction in evaluation :48, datasets provider :108).  ``--mask-type random`` hides
a random walk over the patch grid, ``row`` a band of patch rows; ``--mask-factor`` scales the hidden area.  Data as in
``pretrain_vision_classify.py`` (labels unused).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import pretrain_vision_classify as base  # noqa: E402
from megatron_lm_b200.models.vision import VitInpaintingModel, psnr, random_patch_mask, ssim  # noqa: E402
from megatron_lm_b200.models.vision_backbones import MitInpaintingModel  # noqa: E402
from megatron_lm_b200.parallel import state  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    if state.get_pipeline_model_parallel_world_size() > 1:
        raise NotImplementedError("the in-painting model is trained without pipeline parallelism")
    print_rank_0(f"building the {args.vision_backbone_type} in-painting model ...")
    if args.vision_backbone_type == "mit":
        if args.tensor_model_parallel_size > 1:
            raise NotImplementedError("the MiT backbone is data parallel only")
        dp = state.get_data_parallel_group() if state.get_data_parallel_world_size() > 1 else None
        return MitInpaintingModel(config, args.img_h, args.img_w, args.patch_dim, sync_group=dp)
    if args.vision_backbone_type != "vit":
        raise ValueError(f"no in-painting model on the {args.vision_backbone_type} backbone (vit or mit)")
    return VitInpaintingModel(config, args.img_h, args.img_w, args.patch_dim)


def get_batch(data_iterator):
    args = get_args()
    images, _ = base.get_batch(data_iterator)
    # the same mask on every tensor-parallel rank: drawn from a generator seeded by the step and data-parallel rank
    g = torch.Generator().manual_seed(args.seed + 7919 * getattr(args, "curr_iteration", 0)
                                      + 104729 * state.get_data_parallel_rank() + _COUNTER[0])
    _COUNTER[0] += 1
    mask = random_patch_mask(images.shape[0], args.img_h, args.img_w, args.patch_dim, args.mask_factor, args.mask_type, g)
    mask = mask.to(images.device, images.dtype)
    return images, mask


_COUNTER = [0]


def forward_step(data_iterator, model):
    images, mask = get_batch(data_iterator)
    masked = images * (1 - mask)
    training = model.training

    def loss_func(output):
        out = output.float()
        hidden = mask.float().expand_as(out)
        loss = ((out - images.float()) * hidden).pow(2).sum() / hidden.sum().clamp(min=1.0)
        validate_loss(loss, get_args())
        report = {"loss": loss.detach()}
        if not training:
            full = out * hidden + images.float() * (1 - hidden)        # visible pixels are copied through
            report["psnr"] = psnr(full, images).detach()
            report["ssim"] = ssim(full, images).detach()
        return loss, report
    return model(masked), loss_func


if __name__ == "__main__":
    pretrain(base.train_valid_test_datasets_provider, model_provider, forward_step,
             args_defaults={"tokenizer_type": "NullTokenizer", "vocab_size": 8})
