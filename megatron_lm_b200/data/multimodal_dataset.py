"""Mock image + text dataset for the vision-language program.

Reference: megatron/core/datasets/multimodal_dataset.py (``MultimodalDatasetConfig`` :12 - image size and a
preprocessing hook on top of the GPT dataset configuration; ``MockMultimodalDataset`` :35 - the mock GPT sample with a
random image attached, passed through ``preprocess_func``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

import numpy as np
import torch

from .gpt_dataset import GPTDatasetConfig, MockGPTDataset


@dataclass
class MultimodalDatasetConfig(GPTDatasetConfig):
    image_h: Optional[int] = None
    image_w: Optional[int] = None
    preprocess_func: Optional[Callable[[Dict[str, torch.Tensor]], Dict[str, torch.Tensor]]] = None

    def __post_init__(self):
        super().__post_init__()
        if self.image_h is None or self.image_w is None:
            raise ValueError("MultimodalDatasetConfig needs image_h and image_w")
        if self.preprocess_func is None:
            raise ValueError("MultimodalDatasetConfig needs a preprocess_func (it inserts the image tokens)")


class MockMultimodalDataset(MockGPTDataset):
    """The mock text sample of the GPT dataset plus a reproducible random image [3, image_h, image_w] in [0, 1);
    the configuration's ``preprocess_func`` turns the pair into what the model's forward step expects."""

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        sample = super().__getitem__(idx)
        rng = np.random.RandomState((self.config.random_seed + int(idx)) % (2 ** 32))
        sample["image"] = torch.from_numpy(rng.random_sample((3, self.config.image_h, self.config.image_w))
                                           .astype(np.float32))
        return self.config.preprocess_func(sample)
