"""Which parts of a model run their GEMMs in 8-bit floating point, and helpers around the 8-bit tensor type
(reference: megatron/core/fp8_utils.py:82 is_float8tensor, :99 dequantize_fp8_tensor, :107 get_fp8_align_size,
:413 get_fp8_context).

The reference wraps a layer's forward in a Transformer-Engine autocast context; here the linear layers decide per
call (``parallel/layers.py``: the ``config.fp8`` format and the module's ``fp8_eligible`` mark), so the per-layer
choice is a mark put on the layer's linears when it is built.
"""
from __future__ import annotations

from contextlib import contextmanager

import torch

from .ops.fp8 import Fp8Tensor


def is_float8tensor(t) -> bool:
    return isinstance(t, Fp8Tensor) or (torch.is_tensor(t) and t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2))


def dequantize_fp8_tensor(t) -> torch.Tensor:
    if isinstance(t, Fp8Tensor):
        return t.dequantize()
    return t.float()


def get_fp8_align_size(fp8_recipe=None) -> int:
    """Token counts per expert are padded to this multiple before an 8-bit grouped GEMM: 32 for the block-scaled
    recipe (one scale per 32 elements), 16 otherwise (the tensor-core tile's K granularity for 8-bit operands)."""
    return 32 if str(fp8_recipe or "").endswith("mxfp8") else 16


def layer_runs_in_fp8(config, layer_no: int) -> bool:
    """``layer_no`` is the 0-based index over the whole model.  With ``first_last_layers_bf16`` the first
    ``num_layers_at_start_in_bf16`` and last ``num_layers_at_end_in_bf16`` layers stay in 16 bits."""
    if not getattr(config, "fp8", None):
        return False
    if layer_no >= 0 and getattr(config, "first_last_layers_bf16", False):
        if layer_no < config.num_layers_at_start_in_bf16:
            return False
        if layer_no >= config.num_layers - config.num_layers_at_end_in_bf16:
            return False
    return True


def mark_layer_precision(layer: torch.nn.Module, config, layer_no: int) -> bool:
    """Marks every linear of ``layer`` as eligible for the 8-bit path or not; returns the choice."""
    on = layer_runs_in_fp8(config, layer_no)
    if getattr(config, "fp8", None) and not on:
        for m in layer.modules():
            if hasattr(m, "weight") and hasattr(m, "config"):
                m.fp8_eligible = False
    return on


@contextmanager
def get_fp8_context(config, layer_no: int = -1, is_init: bool = False):
    """Context form of the same choice, for code written against the reference's API: inside it
    ``config.fp8`` reads as None when ``layer_no`` is a 16-bit layer."""
    if layer_runs_in_fp8(config, layer_no) or not getattr(config, "fp8", None):
        yield
        return
    saved, config.fp8 = config.fp8, None
    try:
        yield
    finally:
        config.fp8 = saved


def prepare_model_for_fp8_inference(model: torch.nn.Module, fp8_format: str = "e4m3", recipe: str = "tensorwise"):
    """Switch the transformer-layer linears of a (bf16 / fp16) model to the FP8 GEMM path for inference: the config
    is marked, every eligible linear keeps a cached FP8 image of its weight (quantised once, since weights no longer
    change), and token counts that the 8-bit tensor-core path cannot take (not a multiple of 16, e.g. single-token
    decoding) fall back to 16 bits by themselves.  Returns the number of linears switched
    (reference: megatron/core/fp8_utils.py:604 ``prepare_model_for_fp8_inference``, which pads such inputs instead)."""
    from .parallel.layers import ColumnParallelLinear, RowParallelLinear
    n = 0
    for mod in model.modules():
        cfg = getattr(mod, "config", None)
        if cfg is not None and hasattr(cfg, "fp8"):
            cfg.fp8, cfg.fp8_recipe = fp8_format, recipe
        if isinstance(mod, (ColumnParallelLinear, RowParallelLinear)) and getattr(mod, "fp8_eligible", True) \
                and mod.weight is not None and mod.weight.shape[0] % 16 == 0 and mod.weight.shape[1] % 16 == 0:
            mod.weight.requires_grad_(False)
            n += 1
    model.eval()
    return n
