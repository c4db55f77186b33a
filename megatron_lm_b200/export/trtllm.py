"""Weight conversion to the TensorRT-LLM checkpoint naming, and engine build when the runtime is present.

Reference: megatron/core/export/trtllm/trtllm_helper.py (``TRTLLMHelper`` :39,
``get_trtllm_pretrained_config_and_model_weights`` :188, ``build_and_save_engine`` :445), the layer-name
table trtllm_layers.py and the single-device converter
model_to_trllm_mapping/…/single_device_trtllm_model_weights_converter.py:40.
TensorRT-LLM itself is an external package; without it ``build_and_save_engine`` raises, while the weight
conversion (pure tensor work) runs anywhere.
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional

import torch

from ..checkpoint.convert import _qkv_from_core

_LAYER = {
    "input_layernorm.weight": "input_layernorm.weight",
    "input_layernorm.bias": "input_layernorm.bias",
    "self_attention.linear_proj.weight": "attention.dense.weight",
    "self_attention.linear_proj.bias": "attention.dense.bias",
    "pre_mlp_layernorm.weight": "post_layernorm.weight",
    "pre_mlp_layernorm.bias": "post_layernorm.bias",
    "mlp.linear_fc2.weight": "mlp.proj.weight",
    "mlp.linear_fc2.bias": "mlp.proj.bias",
    "mlp.router.weight": "mlp.router.weight",
}


class TRTLLMHelper:
    def __init__(self, transformer_config, model_type: str = "llama", share_embeddings_and_output_weights: bool = False,
                 activation: str = "swiglu", position_embedding_type: str = "rope", max_position_embeddings: int = 4096,
                 rotary_percentage: float = 1.0, rotary_base: float = 10000.0, seq_len_interpolation_factor=None):
        self.cfg, self.model_type = transformer_config, model_type
        self.share = share_embeddings_and_output_weights
        self.activation, self.pos_type = activation, position_embedding_type
        self.max_pos, self.rot_pct, self.rot_base = max_position_embeddings, rotary_percentage, rotary_base

    def pretrained_config(self, dtype: str = "bfloat16", tp: int = 1, pp: int = 1, vocab_size: Optional[int] = None):
        c = self.cfg
        return {"architecture": {"llama": "LlamaForCausalLM", "gpt": "GPTForCausalLM", "mixtral": "LlamaForCausalLM"}
                .get(self.model_type, "GPTForCausalLM"), "dtype": dtype, "num_hidden_layers": c.num_layers,
                "num_attention_heads": c.num_attention_heads, "num_key_value_heads": c.num_query_groups,
                "hidden_size": c.hidden_size, "intermediate_size": c.ffn_hidden_size, "norm_epsilon": c.layernorm_epsilon,
                "vocab_size": vocab_size, "position_embedding_type": "rope_gpt_neox" if self.pos_type == "rope" else "learned_absolute",
                "max_position_embeddings": self.max_pos, "hidden_act": self.activation, "rotary_base": self.rot_base,
                "rotary_pct": self.rot_pct, "mapping": {"world_size": tp * pp, "tp_size": tp, "pp_size": pp},
                "share_embedding_table": self.share, "moe": {"num_experts": c.num_moe_experts or 0,
                                                             "top_k": c.moe_router_topk if c.num_moe_experts else 0}}

    def convert(self, state_dict: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
        """Full (unpartitioned) core state dict -> TensorRT-LLM names.  Fused QKV is re-ordered to [q ; k ; v]
        and a gated fc1 [gate ; up] is split into ``mlp.gate`` / ``mlp.fc`` the way that runtime expects."""
        c = self.cfg
        out = {}
        seq_experts: Dict[str, Dict[int, torch.Tensor]] = {}
        for k, v in state_dict.items():
            v = v.to(dtype)
            if k == "embedding.word_embeddings.weight":
                out["transformer.vocab_embedding.weight"] = v
            elif k == "embedding.position_embeddings.weight":
                out["transformer.position_embedding.weight"] = v
            elif k.startswith("decoder.final_layernorm."):
                out["transformer.ln_f." + k.rsplit(".", 1)[1]] = v
            elif k == "output_layer.weight":
                out["lm_head.weight"] = v
            else:
                m = re.match(r"^decoder\.layers\.(\d+)\.(.*)$", k)
                if not m:
                    continue
                i, rest = m.group(1), m.group(2)
                base = f"transformer.layers.{i}."
                if rest == "self_attention.linear_qkv.weight":
                    q, kk, vv = _qkv_from_core(v, c.num_attention_heads, c.num_query_groups, c.kv_channels)
                    out[base + "attention.qkv.weight"] = torch.cat((q, kk, vv), 0)
                elif rest == "self_attention.linear_qkv.bias":
                    q, kk, vv = _qkv_from_core(v.unsqueeze(1), c.num_attention_heads, c.num_query_groups, c.kv_channels)
                    out[base + "attention.qkv.bias"] = torch.cat((q, kk, vv), 0).squeeze(1)
                elif rest == "mlp.linear_fc1.weight":
                    if c.gated_linear_unit:
                        gate, up = v.chunk(2, 0)
                        out[base + "mlp.fc.weight"], out[base + "mlp.gate.weight"] = gate, up
                    else:
                        out[base + "mlp.fc.weight"] = v
                elif re.match(r"^mlp\.experts\.local_experts\.\d+\.linear_fc[12]\.weight$", rest):
                    e, which = re.match(r"^mlp\.experts\.local_experts\.(\d+)\.linear_fc([12])", rest).groups()
                    key = base + ("mlp.fc.weight" if which == "1" else "mlp.proj.weight")
                    seq_experts.setdefault(key, {})[int(e)] = v
                elif rest == "mlp.experts.weight1":
                    out[base + "mlp.fc.weight"] = v
                elif rest == "mlp.experts.weight2":
                    out[base + "mlp.proj.weight"] = v
                elif rest in _LAYER:
                    out[base + _LAYER[rest]] = v
        for key, by_e in seq_experts.items():                         # per-expert modules -> one [E, ...] tensor
            out[key] = torch.stack([by_e[e] for e in sorted(by_e)])
        if self.share and "lm_head.weight" not in out:
            out["lm_head.weight"] = out["transformer.vocab_embedding.weight"]
        return out

    # -- tensor / pipeline parallel checkpoints -----------------------------------------------------------------------
    def split_for_mapping(self, weights: Dict[str, torch.Tensor], tp: int = 1, pp: int = 1,
                          use_parallel_embedding: bool = False) -> List[Dict[str, torch.Tensor]]:
        """Converted (full) weights -> one dict per rank of a ``tp x pp`` mapping, rank = pp_rank * tp + tp_rank, in
        the runtime's per-rank layout: fused QKV cut by heads (each rank keeps its own q, k and v heads, again as
        [q ; k ; v]), column-parallel weights along their rows, row-parallel weights along their columns, experts along
        the FFN width, layers dealt to pipeline stages in order with the embedding on the first and the final norm
        and head on the last.  Reference: trtllm_weights_converter/distributed_trtllm_model_weights_converter.py:60-293
        and single_device_trtllm_model_weights_converter.py:300-489."""
        c = self.cfg
        if c.num_layers % pp or c.num_attention_heads % tp or (c.num_query_groups or c.num_attention_heads) % tp:
            raise ValueError("layers must divide by the pipeline size and heads / query groups by the tensor size")
        per_stage = c.num_layers // pp
        ng = c.num_query_groups or c.num_attention_heads
        hn = c.kv_channels or c.hidden_size // c.num_attention_heads
        q_rows, kv_rows = c.num_attention_heads * hn, ng * hn
        ranks: List[Dict[str, torch.Tensor]] = [dict() for _ in range(tp * pp)]

        def cut(name, v, t):
            if name.endswith("attention.qkv.weight") or name.endswith("attention.qkv.bias"):
                q, k, vv = v[:q_rows], v[q_rows:q_rows + kv_rows], v[q_rows + kv_rows:]
                return torch.cat([x.chunk(tp, 0)[t] for x in (q, k, vv)], 0)
            if name.endswith(("mlp.fc.weight", "mlp.gate.weight", "mlp.fc.bias", "mlp.gate.bias")) and v.dim() <= 2:
                return v.chunk(tp, 0)[t]
            if name.endswith(("attention.dense.weight", "mlp.proj.weight")) and v.dim() == 2:
                return v.chunk(tp, 1)[t]
            if v.dim() == 3 and name.endswith("mlp.fc.weight"):        # experts [E, (2)f, h]
                if c.gated_linear_unit:
                    g, u = v.chunk(2, 1)
                    return torch.cat((g.chunk(tp, 1)[t], u.chunk(tp, 1)[t]), 1)
                return v.chunk(tp, 1)[t]
            if v.dim() == 3 and name.endswith("mlp.proj.weight"):      # experts [E, h, f]
                return v.chunk(tp, 2)[t]
            if name == "lm_head.weight":
                return v.chunk(tp, 0)[t]
            if name == "transformer.vocab_embedding.weight" and use_parallel_embedding:
                return v.chunk(tp, 0)[t]
            return v
        for name, v in weights.items():
            m = re.match(r"^transformer\.layers\.(\d+)\.(.*)$", name)
            if m:
                layer = int(m.group(1))
                stages = [layer // per_stage]
                out_name = f"transformer.layers.{layer % per_stage}.{m.group(2)}" if pp > 1 else name
            elif name.startswith(("transformer.vocab_embedding", "transformer.position_embedding")):
                stages, out_name = [0], name
            else:                                                     # final norm, head
                stages, out_name = [pp - 1], name
            for st in stages:
                for t in range(tp):
                    ranks[st * tp + t][out_name] = cut(name, v, t).contiguous() if tp > 1 else v
        return ranks

    def fp8_scaling_factors(self, model) -> Dict[str, torch.Tensor]:
        """Scaling factors of a model quantised by ``post_training.ptq`` (per-tensor FP8) under the runtime's names:
        ``...weights_scaling_factor`` and ``...activation_scaling_factor`` = range / 448 per linear (reference:
        single_device_trtllm_model_weights_converter.py:60-120, scales taken from the FP8 metadata of the layers)."""
        names = {"self_attention.linear_qkv": "attention.qkv", "self_attention.linear_proj": "attention.dense",
                 "mlp.linear_fc1": "mlp.fc", "mlp.linear_fc2": "mlp.proj"}
        out: Dict[str, torch.Tensor] = {}
        for mod_name, mod in model.named_modules():
            m = re.match(r"^(?:.*\.)?decoder\.layers\.(\d+)\.(self_attention\.linear_qkv|self_attention\.linear_proj|"
                         r"mlp\.linear_fc1|mlp\.linear_fc2)$", mod_name)
            if not m or not getattr(mod, "ptq", False) or not hasattr(mod, "weight_quantizer"):
                continue
            base = f"transformer.layers.{m.group(1)}.{names[m.group(2)]}."
            wq, iq = mod.weight_quantizer, mod.input_quantizer
            if wq.spec.kind != "fp8" or wq.spec.block is not None:
                continue
            if getattr(mod, "weight_scale", None) is not None and mod.weight is None:
                out[base + "weights_scaling_factor"] = mod.weight_scale.reshape(1).float()
            elif wq.amax is not None:
                out[base + "weights_scaling_factor"] = (wq.amax.float() / 448.0).reshape(1)
            if iq.amax is not None:
                out[base + "activation_scaling_factor"] = (iq.amax.float() / 448.0).reshape(1)
            if m.group(2) == "mlp.linear_fc1" and self.cfg.gated_linear_unit:
                for k in ("weights_scaling_factor", "activation_scaling_factor"):
                    if base + k in out:
                        out[base.replace("mlp.fc.", "mlp.gate.") + k] = out[base + k]
        return out

    def save_checkpoint(self, out_dir: str, weights_by_rank: List[Dict[str, torch.Tensor]], config: dict) -> List[str]:
        """``config.json`` + one weight file per rank (``rank<N>.safetensors`` when that package is importable, else
        ``rank<N>.pt``): the checkpoint directory the runtime's engine builder reads."""
        import json
        import os
        os.makedirs(out_dir, exist_ok=True)
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(config, f, indent=2)
        files = []
        for r, w in enumerate(weights_by_rank):
            try:
                from safetensors.torch import save_file
                path = os.path.join(out_dir, f"rank{r}.safetensors")
                save_file({k: v.contiguous().clone() for k, v in w.items()}, path)
            except ImportError:
                path = os.path.join(out_dir, f"rank{r}.pt")
                torch.save(w, path)
            files.append(path)
        return files

    def build_and_save_engine(self, engine_dir: str, weights: Dict[str, torch.Tensor], config: dict, **build_kw):
        try:
            import tensorrt_llm  # noqa: F401
        except ImportError as e:
            raise RuntimeError("TensorRT-LLM is not installed; the converted weights and config can be saved with "
                               "torch.save / json and built on a machine that has it") from e
        from tensorrt_llm.builder import BuildConfig, build
        from tensorrt_llm.models import PretrainedConfig, MODEL_MAP
        pc = PretrainedConfig.from_dict(config)
        model = MODEL_MAP[config["architecture"]].from_config(pc)
        model.load(weights)
        engine = build(model, BuildConfig(**build_kw))
        engine.save(engine_dir)
