"""Enumerations shared by the model code (reference: megatron/core/transformer/enums.py:8-70,
megatron/core/enums.py)."""
from __future__ import annotations

import enum


class ModelType(enum.Enum):
    encoder_or_decoder = 1
    encoder_and_decoder = 2
    retro_encoder = 3
    retro_decoder = 4


class LayerType(enum.Enum):
    """What a pipeline stage of an explicit layer layout holds."""
    embedding = 1
    loss = 2
    encoder = 3
    decoder = 4
    mtp = 5


class AttnType(enum.Enum):
    self_attn = 1
    cross_attn = 2


class AttnMaskType(enum.Enum):
    padding = 1
    causal = 2
    no_mask = 3
    padding_causal = 4
    arbitrary = 5


class AttnBackend(enum.Enum):
    """Which attention implementation a config asks for.  ``flash`` / ``fused`` / ``auto`` all select the sm_100a
    flash kernel of this library when the shape is supported; ``unfused`` and ``local`` select the masked softmax
    path in plain PyTorch."""
    flash = 1
    fused = 2
    unfused = 3
    local = 4
    auto = 5


class Fp8Recipe(str, enum.Enum):
    delayed = "delayed"
    tensorwise = "tensorwise"
    mxfp8 = "mxfp8"
    blockwise = "blockwise"
