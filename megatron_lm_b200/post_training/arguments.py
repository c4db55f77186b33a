"""Command-line flags of the post-training programs (quantisation, distillation).

Reference: megatron/post_training/arguments.py:4-120 (``add_modelopt_args``: the ``--export-*`` family).  The names,
defaults and choices are the reference's, so launch scripts carry over; flags that select a code path of the
external library with no counterpart here are accepted and reported by ``unsupported_set``.
"""
from __future__ import annotations

from typing import List

QUANT_CHOICES = ["int8_sq", "fp8", "fp8_real_quant", "fp8_blockwise", "fp8_blockwise_real_quant", "fp8_blockwise_32",
                 "int4_awq", "w4a8_awq", "nvfp4", "None"]

_NO_EFFECT = {
    "export_legacy_megatron": False,
    "export_te_mcore_model": False,
    "export_force_local_attention": False,
    "export_kv_cache_quant": False,
    "finetune_hf_dataset": None,
    "export_moe_apply_probs_on_input": False,
}


def add_modelopt_args(parser):
    g = parser.add_argument_group(title="post-training")
    g.add_argument("--export-model-type", default="GPTModel", choices=["GPTModel", "MambaModel"])
    g.add_argument("--export-legacy-megatron", action="store_true")
    g.add_argument("--export-te-mcore-model", action="store_true")
    g.add_argument("--export-force-local-attention", action="store_true")
    g.add_argument("--export-kv-cache-quant", action="store_true")
    g.add_argument("--export-real-quant-cfg", default="None",
                   choices=["fp8_real_quant", "fp8_blockwise_real_quant", "None"],
                   help="hold the linears' weights as FP8 values plus scales")
    g.add_argument("--export-quant-cfg", default=None, choices=QUANT_CHOICES,
                   help="post-training quantisation recipe")
    g.add_argument("--export-kd-cfg", default=None, help="distillation configuration (YAML)")
    g.add_argument("--export-kd-teacher-load", default=None, help="checkpoint of the distillation teacher")
    g.add_argument("--export-kd-teacher-ckpt-format", default=None, choices=["torch", "torch_dist", "zarr", "torch_dcp"])
    g.add_argument("--finetune-hf-dataset", default=None)
    g.add_argument("--finetune-data-split", default="train")
    g.add_argument("--export-qk-l2-norm", action="store_true", help="L2 normalisation of queries and keys")
    g.add_argument("--export-moe-apply-probs-on-input", action="store_true")
    return parser


def modelopt_args_enabled(args) -> bool:
    """True when a run asks for quantisation, compressed weights or distillation."""
    return any([getattr(args, "export_quant_cfg", None) not in (None, "None"),
                getattr(args, "export_real_quant_cfg", "None") not in (None, "None"),
                getattr(args, "export_kd_cfg", None) is not None,
                getattr(args, "export_kd_teacher_load", None) is not None])


def unsupported_set(args) -> List[str]:
    """Flags of the family that were given a non-default value but change nothing here."""
    return [k for k, d in _NO_EFFECT.items() if getattr(args, k, d) != d]
