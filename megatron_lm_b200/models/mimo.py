"""MIMO: a language model fed by any number of modality encoders.

Reference: megatron/core/models/mimo/model/base.py (``MimoModel`` :20, ``align_embeddings_by_token_positions``
:93, forward :211) and mimo/submodules/base.py (``ModalitySubmodules``).  Each modality has encoders whose
outputs are concatenated, then projected to the language model's width; the projected rows replace the
language embeddings at the positions of that modality's special token.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn


class ModalitySubmodules(nn.Module):
    def __init__(self, encoders: Optional[Dict[str, nn.Module]] = None, decoders: Optional[Dict[str, nn.Module]] = None,
                 input_projections=None, output_projections=None):
        super().__init__()
        self.encoders = nn.ModuleDict(encoders or {})
        self.decoders = nn.ModuleDict(decoders or {})
        self.input_projections = nn.ModuleList(input_projections or [])
        self.output_projections = nn.ModuleList(output_projections or [])

    def encode(self, inputs: Dict[str, dict]):
        outs = []
        for name, enc in self.encoders.items():
            if name not in inputs:
                continue
            o = enc(**inputs[name])
            outs.append(o.reshape(-1, o.shape[-1]))
        return outs

    def forward(self, encoder_inputs: Dict[str, dict]):
        outs = self.encode(encoder_inputs)
        if not outs:
            return None
        x = torch.cat(outs, dim=0)
        for proj in self.input_projections:
            x = proj(x)
        return x                                                            # [n_embeddings, h]


class MimoModel(nn.Module):
    def __init__(self, language_model: nn.Module, modality_submodules: Dict[str, ModalitySubmodules],
                 special_token_ids: Dict[str, int]):
        super().__init__()
        self.language_model = language_model
        self.modality_submodules = nn.ModuleDict(modality_submodules)
        self.special_token_ids = dict(special_token_ids)

    def set_input_tensor(self, t):
        self.language_model.set_input_tensor(t)

    def get_text_embeddings(self, input_ids, position_ids):
        text_mask = torch.ones_like(input_ids, dtype=torch.bool)
        for tok in self.special_token_ids.values():
            text_mask &= input_ids != tok
        ids = torch.where(text_mask, input_ids, torch.zeros_like(input_ids))
        emb = self.language_model.embedding(ids, position_ids).transpose(0, 1)     # [b, s, h]
        return emb, text_mask

    def align_embeddings_by_token_positions(self, modality_embeddings: Dict[str, torch.Tensor], input_ids, text_emb):
        out = text_emb.clone()
        for name, emb in modality_embeddings.items():
            mask = input_ids == self.special_token_ids[name]
            n = int(mask.sum())
            if n != emb.shape[0]:
                raise ValueError(f"{name}: {n} placeholder tokens but {emb.shape[0]} embeddings")
            out[mask] = emb.to(out.dtype)
        return out.transpose(0, 1).contiguous()                             # [s, b, h]

    def forward(self, input_ids, position_ids=None, attention_mask=None, loss_mask=None, labels=None,
                modality_inputs: Optional[Dict[str, Dict[str, dict]]] = None):
        embs = {}
        for name, sub in self.modality_submodules.items():
            if modality_inputs and name in modality_inputs:
                e = sub(modality_inputs[name])
                if e is not None:
                    embs[name] = e
        text_emb, _ = self.get_text_embeddings(input_ids, position_ids)
        dec_in = self.align_embeddings_by_token_positions(embs, input_ids, text_emb)
        out = self.language_model(None, position_ids, attention_mask, decoder_input=dec_in, labels=labels)
        return out, loss_mask
