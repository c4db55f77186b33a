"""LLaVA-style vision-language model: vision encoder -> projector -> language model, with image
embeddings spliced into the text sequence at image-token positions.

Reference: megatron/core/models/multimodal/llava_model.py (``LLaVAModel`` :53, ``_preprocess_data``
:386, forward :745).  Text tokens keep their labels and loss mask; positions covered by image
embeddings are masked out of the loss, except that the label of the token after the image is kept.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..config import TransformerConfig
from .gpt import GPTModel
from .vision import CLIPViTModel, MultimodalProjector, RADIOViTModel, get_num_image_embeddings

IGNORE_INDEX = -100
DEFAULT_IMAGE_TOKEN_INDEX = -200
IMAGE_TOKEN = "<image>"


class LLaVAModel(nn.Module):
    def __init__(self, language_transformer_config: TransformerConfig, language_vocab_size: int,
                 language_max_sequence_length: int, vision_transformer_config: TransformerConfig,
                 vision_projection_config: TransformerConfig, vision_projection_type: str = "mlp",
                 drop_vision_class_token: bool = False, img_h: int = 336, img_w: int = 336, patch_dim: int = 14,
                 language_position_embedding_type: str = "learned_absolute", pre_process: bool = True,
                 post_process: bool = True, add_encoder: bool = True, add_decoder: bool = True,
                 vision_model_type: str = "clip", image_token_index: int = DEFAULT_IMAGE_TOKEN_INDEX,
                 parallel_output: bool = True, share_embeddings_and_output_weights: bool = False,
                 language_transformer_layer_spec=None, vision_transformer_layer_spec=None,
                 vision_projection_layer_spec=None, allow_missing_vision_projection_checkpoint: bool = False):
        super().__init__()
        self.config = language_transformer_config      # the training loop reads the model's config from here
        self.pre_process, self.post_process = pre_process, post_process
        self.add_encoder, self.add_decoder = add_encoder, add_decoder
        self.image_token_index = image_token_index
        self.drop_class = drop_vision_class_token
        self.max_len = language_max_sequence_length
        self.vision_model = self.vision_projection = self.language_model = None
        if add_encoder:
            if vision_model_type == "radio":
                self.vision_model = RADIOViTModel(vision_transformer_config, img_h=img_h, img_w=img_w,
                                                  patch_dim=patch_dim)
            else:
                self.vision_model = CLIPViTModel(vision_transformer_config, img_h=img_h, img_w=img_w,
                                                 patch_dim=patch_dim, model_subtype=vision_model_type)
            self.vision_projection = MultimodalProjector(vision_projection_config, None, vision_projection_type,
                                                         vision_transformer_config.hidden_size)
            self.class_len = self.vision_model.class_token_len
        if add_decoder:
            self.language_model = GPTModel(language_transformer_config, language_vocab_size,
                                           language_max_sequence_length, pre_process, post_process,
                                           parallel_output=parallel_output,
                                           share_embeddings_and_output_weights=share_embeddings_and_output_weights,
                                           position_embedding_type=language_position_embedding_type)
        self.img_seq_len = get_num_image_embeddings(img_h, img_w, patch_dim, vision_model_type,
                                                    drop_vision_class_token,
                                                    getattr(self.vision_model, "class_token_len", 1) if add_encoder else 1)

    def set_input_tensor(self, t):
        if isinstance(t, (list, tuple)):
            t = t[0]
        if self.add_decoder:
            self.language_model.set_input_tensor(t)
        elif self.add_encoder:
            self.vision_model.set_input_tensor(t)

    def freeze(self, freeze_language_model: bool, freeze_vision_model: bool, freeze_vision_projection: bool):
        for flag, mod in ((freeze_language_model, self.language_model), (freeze_vision_model, self.vision_model),
                          (freeze_vision_projection, self.vision_projection)):
            if flag and mod is not None:
                for p in mod.parameters():
                    p.requires_grad = False

    def _splice(self, image_embeddings, text_embeddings, input_ids, labels, loss_mask, num_image_tiles):
        """image_embeddings [tiles, n_img, h]; text_embeddings [b, s_text, h].  Returns combined
        embeddings [b, S, h] with labels / loss mask [b, S] (right-padded to the longest sample)."""
        b, s_text = input_ids.shape
        n_img = image_embeddings.shape[1]
        outs, out_labels, out_masks = [], [], []
        tile = 0
        img_idx = 0
        for i in range(b):
            pieces, lab, msk = [], [], []
            pos = (input_ids[i] == self.image_token_index).nonzero().flatten().tolist()
            prev = 0
            for p_ in pos:
                pieces.append(text_embeddings[i, prev:p_])
                tiles = int(num_image_tiles[img_idx]) if num_image_tiles is not None else 1
                emb = image_embeddings[tile:tile + tiles].reshape(tiles * n_img, -1)
                pieces.append(emb)
                if labels is not None:
                    lab.append(labels[i, prev:p_])
                    msk.append(loss_mask[i, prev:p_])
                    il = torch.full((tiles * n_img,), IGNORE_INDEX, dtype=labels.dtype, device=labels.device)
                    im = torch.zeros(tiles * n_img, dtype=loss_mask.dtype, device=loss_mask.device)
                    # the last image embedding predicts the first text token after the image
                    il[-1] = labels[i, p_]
                    im[-1] = loss_mask[i, p_]
                    lab.append(il)
                    msk.append(im)
                tile += tiles
                img_idx += 1
                prev = p_ + 1
            pieces.append(text_embeddings[i, prev:])
            if labels is not None:
                lab.append(labels[i, prev:])
                msk.append(loss_mask[i, prev:])
            outs.append(torch.cat(pieces, dim=0)[: self.max_len])
            if labels is not None:
                out_labels.append(torch.cat(lab)[: self.max_len])
                out_masks.append(torch.cat(msk)[: self.max_len])
        S = max(o.shape[0] for o in outs)
        emb = torch.zeros(b, S, outs[0].shape[-1], dtype=outs[0].dtype, device=outs[0].device)
        new_labels = new_mask = None
        if labels is not None:
            new_labels = torch.full((b, S), IGNORE_INDEX, dtype=labels.dtype, device=labels.device)
            new_mask = torch.zeros(b, S, dtype=loss_mask.dtype, device=loss_mask.device)
        for i, o in enumerate(outs):
            emb[i, : o.shape[0]] = o
            if labels is not None:
                new_labels[i, : o.shape[0]] = out_labels[i]
                new_mask[i, : o.shape[0]] = out_masks[i]
        return emb, new_labels, new_mask

    def forward(self, images, input_ids, position_ids=None, attention_mask=None, labels=None, loss_mask=None,
                inference_context=None, num_image_tiles=None, image_token_index=None):
        if image_token_index is not None:
            self.image_token_index = image_token_index
        image_embeddings = None
        if self.add_encoder and images is not None and images.shape[0] > 0:
            feats = self.vision_model(images)                               # [tiles, s_img, hv]
            if self.drop_class and self.class_len:
                feats = feats[:, self.class_len:]
            image_embeddings = self.vision_projection(feats)
        if not self.add_decoder:
            return image_embeddings, loss_mask
        lm = self.language_model
        if not self.pre_process:
            out = lm(None, position_ids, attention_mask, labels=labels, inference_context=inference_context)
            return out, loss_mask
        ids_text = input_ids.clone()
        ids_text[ids_text == self.image_token_index] = 0
        text_emb = lm.embedding(ids_text, position_ids).transpose(0, 1)       # [b, s, h]
        if image_embeddings is None:
            emb, new_labels, new_mask = text_emb, labels, loss_mask
        else:
            if labels is not None and loss_mask is None:
                loss_mask = torch.ones_like(labels, dtype=torch.float32)
            emb, new_labels, new_mask = self._splice(image_embeddings.to(text_emb.dtype), text_emb, input_ids, labels,
                                                     loss_mask, num_image_tiles)
        dec_in = emb.transpose(0, 1).contiguous()
        lab_in = None
        if new_labels is not None:
            lab_in = new_labels.clone()
            lab_in[lab_in == IGNORE_INDEX] = 0
        out = lm(None, None, attention_mask, decoder_input=dec_in, labels=lab_in, inference_context=inference_context)
        if labels is None:
            return out
        return out, new_mask
