#!/usr/bin/env python
"""Self-supervised pre-training of a vision transformer with DINO (self-distillation with no labels).

Reference: pretrain_vision_dino.py (model provider :21, loss through the model's ``dino_loss`` in training and a k-NN
monitor on the teacher's features in evaluation :44, datasets provider :88), megatron/legacy/model/vision/dino.py,
knn_monitor.py, and the multi-crop augmentation of legacy/data/vit_dataset.py (two global crops at the full size,
``--dino-local-crops-number`` local crops of ``--dino-local-img-size``).  The momentum teacher follows the student
after every optimizer step; the prototype layer is frozen for the first ``--dino-freeze-last-layer`` epochs
(``--iter-per-epoch`` iterations each); the teacher temperature warms up over ``--dino-warmup-teacher-temp-epochs``.
Data as in ``pretrain_vision_classify.py``; labels are used by the k-NN monitor only.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import pretrain_vision_classify as base  # noqa: E402
from megatron_lm_b200.models.vision import DINOPretrainModel, knn_predict  # noqa: E402
from megatron_lm_b200.parallel import state  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.batch import broadcast_data  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def add_dino_args(parser):
    g = parser.add_argument_group(title="dino")
    g.add_argument("--dino-out-dim", type=int, default=65536, help="number of prototypes of the projection head")
    g.add_argument("--knn-bank-size", type=int, default=256, help="training images in the k-NN monitor's feature bank")
    return parser


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    if state.get_pipeline_model_parallel_world_size() > 1 or state.get_tensor_model_parallel_world_size() > 1:
        raise NotImplementedError("DINO pre-training is data parallel only")
    print_rank_0("building the DINO student and teacher ...")
    dp = state.get_data_parallel_group() if state.get_data_parallel_world_size() > 1 else None
    return DINOPretrainModel(
        config, img_h=args.img_h, img_w=args.img_w, patch_dim=args.patch_dim, out_dim=args.dino_out_dim,
        head_hidden=args.dino_head_hidden_size, bottleneck=args.dino_bottleneck_size,
        norm_last_layer=args.dino_norm_last_layer, local_crops=args.dino_local_crops_number,
        warmup_teacher_temp=args.dino_warmup_teacher_temp, teacher_temp=args.dino_teacher_temp,
        warmup_teacher_temp_iters=args.dino_warmup_teacher_temp_epochs * args.iter_per_epoch,
        total_iters=args.train_iters, freeze_last_layer_iters=int(args.dino_freeze_last_layer * args.iter_per_epoch),
        dp_group=dp, backbone_type=args.vision_backbone_type, swin_type=args.swin_backbone_type)


def _crop(img: torch.Tensor, scale, out_hw, rng) -> torch.Tensor:
    """Random-area crop (area fraction in ``scale``), resized to ``out_hw``, random horizontal flip, brightness
    jitter."""
    _, h, w = img.shape
    frac = rng.uniform(*scale)
    ch, cw = max(int(round(h * frac ** 0.5)), 4), max(int(round(w * frac ** 0.5)), 4)
    y0, x0 = rng.randint(0, h - ch + 1), rng.randint(0, w - cw + 1)
    c = img[:, y0:y0 + ch, x0:x0 + cw].unsqueeze(0)
    c = F.interpolate(c, size=out_hw, mode="bilinear", align_corners=False)[0]
    if rng.rand() < 0.5:
        c = c.flip(-1)
    return c * float(rng.uniform(0.8, 1.2))


class MultiCropDataset(torch.utils.data.Dataset):
    """Wraps an image dataset: every sample becomes two global and N local crops (training) or the plain image."""

    def __init__(self, inner, local_crops, local_size, train, seed):
        self.inner, self.n_local, self.local, self.train, self.seed = inner, local_crops, local_size, train, seed

    def __len__(self):
        return len(self.inner)

    def __getitem__(self, i):
        item = self.inner[i]
        img = torch.from_numpy(np.ascontiguousarray(item["image"]))
        out = {"label": item["label"]}
        if not self.train:
            out["crop0"] = img.numpy()
            return out
        rng = np.random.RandomState((self.seed + 7 * i) % (2 ** 32))
        hw = img.shape[-2:]
        out["crop0"] = _crop(img, (0.4, 1.0), hw, rng).numpy()
        out["crop1"] = _crop(img, (0.4, 1.0), hw, rng).numpy()
        for k in range(self.n_local):
            out[f"crop{2 + k}"] = _crop(img, (0.05, 0.4), (self.local, self.local), rng).numpy()
        return out


def get_batch(data_iterator, training):
    args = get_args()
    data = next(data_iterator) if data_iterator is not None else None
    n = 2 + args.dino_local_crops_number if training else 1
    dt = torch.bfloat16 if args.bf16 else (torch.float16 if args.fp16 else torch.float32)
    crops = [broadcast_data([f"crop{k}"], data, torch.float32)[f"crop{k}"].to(dt) for k in range(n)]
    labels = broadcast_data(["label"], data, torch.int64)["label"].view(-1).long()
    return crops, labels


_BANK = {}


@torch.no_grad()
def feature_bank(model):
    """Teacher features and labels of the first ``--knn-bank-size`` training images (rebuilt when training moved on)."""
    args = get_args()
    key = getattr(args, "curr_iteration", 0)
    if _BANK.get("key") != key:
        shape = (args.num_channels, args.img_h, args.img_w)
        if args.mock_data or not args.data_path:
            ds = base.MockImageDataset(args.knn_bank_size, args.num_classes, *shape, args.seed)
        else:
            ds = base.ImageFolderDataset(os.path.join(args.data_path[0], "train"), *shape, args.knn_bank_size)
        dev = next(model.parameters()).device
        dt = next(model.parameters()).dtype
        feats, labels = [], []
        for lo in range(0, len(ds), 32):
            items = [ds[i] for i in range(lo, min(lo + 32, len(ds)))]
            x = torch.from_numpy(np.stack([it["image"] for it in items])).to(dev, dt)
            feats.append(F.normalize(model(x)[1].float(), dim=1))
            labels.extend(int(it["label"][0]) for it in items)
        _BANK.update(key=key, bank=torch.cat(feats).t().contiguous(), labels=torch.tensor(labels, device=dev))
    return _BANK["bank"], _BANK["labels"]


def forward_step(data_iterator, model):
    args = get_args()
    from megatron_lm_b200.training.checkpointing import _unwrap
    core = _unwrap(model)
    training = core.training
    crops, labels = get_batch(data_iterator, training)

    def loss_func(output):
        if training:
            student, teacher = output
            loss = core.dino_loss(student, teacher, getattr(args, "curr_iteration", 0))
            validate_loss(loss, args)
            return loss, {"loss": loss.detach()}
        bank, bank_labels = feature_bank(core)
        feat = F.normalize(output[1].float(), dim=1)
        report = {}
        for k in (10, 20):
            pred = knn_predict(feat, bank, bank_labels, args.num_classes, k, 0.07)
            report[f"knn_acc_{k}"] = (pred[:, 0] == labels).float().mean() * 100.0
        zero = feat.sum() * 0.0
        return zero, dict(report, loss=zero.detach())
    if training:
        core.set_iteration(getattr(args, "curr_iteration", 0))
    return model(crops if training else crops[0]), loss_func


def train_valid_test_datasets_provider(num_samples):
    args = get_args()
    sets = base.train_valid_test_datasets_provider(num_samples)
    return tuple(None if s is None else MultiCropDataset(s, args.dino_local_crops_number, args.dino_local_img_size,
                                                        train=(i == 0), seed=args.seed + i)
                 for i, s in enumerate(sets))


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step, extra_args_provider=add_dino_args,
             args_defaults={"tokenizer_type": "NullTokenizer", "vocab_size": 8})
