"""Checkpoint glue for quantised models: the description of the attached quantisers is written beside the model file
and re-applied to a freshly built model before its state dict is loaded.

Reference: megatron/post_training/checkpointing.py:59-157 (``load_modelopt_state`` reads ``modelopt_state`` beside
the checkpoint and restores the model's structure before ``load_modelopt_checkpoint`` fills the weights).
Quantised models are saved in the per-rank ``torch`` format: quantiser ranges and compressed weights are buffers of
the model's state dict, which that format stores whole.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Sequence

from . import ptq

STATE_FILE = "quantizer_state.json"


def has_quantizers(model_chunks: Sequence) -> bool:
    return any(getattr(m, "ptq", False) or hasattr(m, "weight_quantizer")
               for chunk in model_chunks for m in chunk.modules())


def save_quantizer_state(model_chunks: Sequence, directory: str) -> Optional[str]:
    """Write {chunk index: structure} into ``directory`` (the folder of this model-parallel rank's file)."""
    if not has_quantizers(model_chunks):
        return None
    from ..training.checkpointing import _unwrap
    state = {str(i): ptq.quantizer_state(_unwrap(chunk)) for i, chunk in enumerate(model_chunks)}
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, STATE_FILE)
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(state, f)
    os.replace(tmp, path)
    return path


def load_quantizer_state(directory: str) -> Optional[Dict]:
    path = os.path.join(directory, STATE_FILE)
    if not os.path.isfile(path):
        return None
    with open(path) as f:
        return json.load(f)


def maybe_restore_quantizer_state(model_chunks: Sequence, directory: str) -> bool:
    state = load_quantizer_state(directory)
    if state is None:
        return False
    from ..training.checkpointing import _unwrap
    for i, chunk in enumerate(model_chunks):
        ptq.restore_quantizer_state(_unwrap(chunk), state[str(i)])
    return True
