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
from typing import Dict, Optional

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
                elif rest == "mlp.experts.weight1":
                    out[base + "mlp.fc.weight"] = v
                elif rest == "mlp.experts.weight2":
                    out[base + "mlp.proj.weight"] = v
                elif rest in _LAYER:
                    out[base + _LAYER[rest]] = v
        if self.share and "lm_head.weight" not in out:
            out["lm_head.weight"] = out["transformer.vocab_embedding.weight"]
        return out

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
