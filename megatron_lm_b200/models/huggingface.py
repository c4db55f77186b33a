"""Thin adapters that let Hugging Face modules sit where this framework's encoders go.

Reference: megatron/core/models/huggingface/module.py (``HuggingFaceModule`` :9, ``AutoHuggingFaceModel``
:33), clip_model.py:12, qwen_model.py:12, ``build_hf_model`` module.py:84.
"""
from __future__ import annotations

import torch
import torch.nn as nn


class HuggingFaceModule(nn.Module):
    """Base: holds ``self.model`` (a transformers module); no pipeline input plumbing."""

    def __init__(self, config=None):
        super().__init__()
        self.config = config

    def set_input_tensor(self, input_tensor):
        self.input_tensor = input_tensor

    def __setattr__(self, name, value):
        super().__setattr__(name, value)
        if isinstance(value, nn.Module):                      # mark parameters as replicated, never TP-sharded
            for p in value.parameters():
                if not hasattr(p, "tensor_model_parallel"):
                    p.tensor_model_parallel = False


class AutoHuggingFaceModel(HuggingFaceModule):
    def __init__(self, config, model_name_or_config=None):
        super().__init__(config)
        from transformers import AutoConfig, AutoModel
        src = model_name_or_config if model_name_or_config is not None else getattr(config, "huggingface_model_name_or_path")
        if isinstance(src, str):
            self.model = AutoModel.from_pretrained(src)
        else:
            self.model = AutoModel.from_config(src)

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)


class ClipHuggingFaceModel(HuggingFaceModule):
    def __init__(self, config, hf_config=None):
        super().__init__(config)
        from transformers import CLIPVisionConfig, CLIPVisionModel
        self.model = CLIPVisionModel(hf_config) if hf_config is not None else CLIPVisionModel.from_pretrained(
            config.huggingface_model_name_or_path)

    def forward(self, x, attention_mask=None):
        return self.model(x)["last_hidden_state"]


class QwenHuggingFaceModel(HuggingFaceModule):
    def __init__(self, config, hf_config=None):
        super().__init__(config)
        from transformers import AutoModel
        self.model = AutoModel.from_config(hf_config) if hf_config is not None else AutoModel.from_pretrained(
            config.huggingface_model_name_or_path)

    def embedding(self, input_ids, position_ids=None):
        return self.model.get_input_embeddings()(input_ids).transpose(0, 1).contiguous()

    def forward(self, input_ids=None, position_ids=None, attention_mask=None, decoder_input=None, labels=None, **kw):
        if decoder_input is not None:
            out = self.model(inputs_embeds=decoder_input.transpose(0, 1), position_ids=position_ids)
        else:
            out = self.model(input_ids=input_ids, position_ids=position_ids)
        return out["last_hidden_state"]


def build_hf_model(config, model_full_name: str):
    """``"hf://<name>"`` -> adapter chosen by the model family in the name."""
    name = model_full_name.split("hf://")[-1]
    config.huggingface_model_name_or_path = name
    low = name.lower()
    if "clip" in low:
        return ClipHuggingFaceModel(config)
    if "qwen" in low:
        return QwenHuggingFaceModel(config)
    return AutoHuggingFaceModel(config, name)
