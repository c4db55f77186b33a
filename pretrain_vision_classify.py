#!/usr/bin/env python
"""Pre-train a vision transformer as an image classifier.

Reference: pretrain_vision_classify.py (model provider :19, get_batch :47, cross-entropy + accuracy :60, datasets
provider :90).  Data: ``--data-path ROOT`` with ``ROOT/train/<class>/*.npy`` and ``ROOT/val/<class>/*.npy`` (arrays
[c, h, w] or [h, w, c], uint8 or float; image files too when Pillow is importable), or ``--mock-data`` for synthetic
images whose label is a function of their content.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from megatron_lm_b200.models.vision import VitClassificationModel  # noqa: E402
from megatron_lm_b200.models.vision_backbones import MitClassificationModel  # noqa: E402
from megatron_lm_b200.parallel import state  # noqa: E402
from megatron_lm_b200.training.arguments import get_args  # noqa: E402
from megatron_lm_b200.training.batch import broadcast_data  # noqa: E402
from megatron_lm_b200.training.pretrain import pretrain, print_rank_0  # noqa: E402
from megatron_lm_b200.training.resilience import validate_loss  # noqa: E402


def model_provider(pre_process=True, post_process=True, vp_stage=None, config=None):
    args = get_args()
    if state.get_pipeline_model_parallel_world_size() > 1:
        raise NotImplementedError("the vision classifier is trained without pipeline parallelism")
    print_rank_0(f"building the {args.vision_backbone_type} classification model ...")
    if args.vision_backbone_type == "mit":
        _data_parallel_only(args)
        return MitClassificationModel(config, args.num_classes)
    if args.vision_backbone_type != "vit":
        raise ValueError(f"no classification model on the {args.vision_backbone_type} backbone (vit or mit)")
    return VitClassificationModel(config, args.num_classes, args.img_h, args.img_w, args.patch_dim)


def _data_parallel_only(args):
    if args.tensor_model_parallel_size > 1:
        raise NotImplementedError("the MiT and Swin backbones are data parallel only")


class MockImageDataset(torch.utils.data.Dataset):
    """Random images; the label is the quadrant-brightness pattern of the image, so a model can learn it."""

    def __init__(self, n, num_classes, c, h, w, seed):
        self.n, self.k, self.shape, self.seed = n, num_classes, (c, h, w), seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        rng = np.random.RandomState((self.seed + i) % (2 ** 32))
        label = int(rng.randint(0, self.k))
        img = rng.standard_normal(self.shape).astype(np.float32) * 0.1
        c, h, w = self.shape
        img[:, : h // 2, : w // 2] += (label % 2) * 1.0
        img[:, h // 2:, w // 2:] += ((label // 2) % 2) * 1.0
        img[:, : h // 2, w // 2:] += (label / max(self.k - 1, 1)) - 0.5
        return {"image": img, "label": np.asarray([label], dtype=np.int64)}


class ImageFolderDataset(torch.utils.data.Dataset):
    def __init__(self, root, c, h, w, n=0, classes_fraction=1.0, data_per_class_fraction=1.0):
        """``classes_fraction`` keeps the first part of the (sorted) classes, ``data_per_class_fraction`` the first
        part of every class's (sorted) files (reference: megatron/legacy/data/image_folder.py:80-140)."""
        self.c, self.h, self.w = c, h, w
        classes = sorted(d for d in os.listdir(root) if os.path.isdir(os.path.join(root, d)))
        classes = classes[:max(1, int(len(classes) * classes_fraction))]
        self.classes = classes
        self.items = []
        for i, k in enumerate(classes):
            files = sorted(os.listdir(os.path.join(root, k)))
            files = files[:max(1, int(len(files) * data_per_class_fraction))]
            self.items.extend((os.path.join(root, k, f), i) for f in files)
        if not self.items:
            raise ValueError(f"no images under {root}")
        self.n = n or len(self.items)

    def __len__(self):
        return self.n

    def _load(self, path):
        if path.endswith(".npy"):
            a = np.load(path)
        else:
            from PIL import Image
            a = np.asarray(Image.open(path).convert("RGB"))
        a = a.astype(np.float32) / (255.0 if a.dtype == np.uint8 else 1.0)
        if a.ndim == 3 and a.shape[0] != self.c:
            a = a.transpose(2, 0, 1)
        t = torch.from_numpy(np.ascontiguousarray(a)).unsqueeze(0)
        if t.shape[-2:] != (self.h, self.w):
            t = F.interpolate(t, size=(self.h, self.w), mode="bilinear", align_corners=False)
        return t[0].numpy()

    def __getitem__(self, i):
        path, label = self.items[i % len(self.items)]
        return {"image": self._load(path), "label": np.asarray([label], dtype=np.int64)}


def get_batch(data_iterator):
    args = get_args()
    data = next(data_iterator) if data_iterator is not None else None
    imgs = broadcast_data(["image"], data, torch.float32)["image"]
    labels = broadcast_data(["label"], data, torch.int64)["label"]
    dt = torch.bfloat16 if args.bf16 else (torch.float16 if args.fp16 else torch.float32)
    return imgs.to(dt), labels.view(-1).long()


def forward_step(data_iterator, model):
    images, labels = get_batch(data_iterator)

    def loss_func(logits):
        loss = F.cross_entropy(logits.float(), labels)
        validate_loss(loss, get_args())
        acc = (logits.argmax(dim=-1) == labels).float().mean() * 100.0
        return loss, {"loss": loss.detach(), "accuracy": acc.detach()}
    return model(images), loss_func


def train_valid_test_datasets_provider(num_samples):
    args = get_args()
    shape = (args.num_channels, args.img_h, args.img_w)
    if args.mock_data or not args.data_path:
        return tuple(MockImageDataset(n, args.num_classes, *shape, args.seed + 1000 * i) if n else None
                     for i, n in enumerate(num_samples))
    root = args.data_path[0]
    out = []
    for n, sub in zip(num_samples, ("train", "val", "test")):
        d = os.path.join(root, sub)
        out.append(ImageFolderDataset(d, *shape, n, getattr(args, "classes_fraction", 1.0),
                                      getattr(args, "data_per_class_fraction", 1.0) if sub == "train" else 1.0)
                   if n and os.path.isdir(d) else None)
    return tuple(out)


if __name__ == "__main__":
    pretrain(train_valid_test_datasets_provider, model_provider, forward_step,
             args_defaults={"tokenizer_type": "NullTokenizer", "vocab_size": 8})
