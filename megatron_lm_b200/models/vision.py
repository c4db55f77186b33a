"""Vision transformers and the projector that feeds them to a language model.

Reference: megatron/core/models/vision/clip_vit_model.py (``CLIPViTModel`` :26,
``get_num_image_embeddings`` :224), vision/radio.py (``RADIOViTModel`` :29),
vision/multimodal_projector.py (``MultimodalProjector`` :18), vision/vit_layer_specs.py.
Images [b, 3, H, W] are cut into patches and embedded by one GEMM (the strided conv of the reference is
a linear map on the unfolded patches), prefixed with class tokens, given learned positions and run
through a bidirectional transformer block.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import TransformerConfig
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear, _device
from .transformer import MLP, Norm, TransformerBlock


def get_num_image_embeddings(img_h: int, img_w: int, patch_dim: int, vision_model_type: str = "clip",
                             disable_vision_class_token: bool = False, class_token_len: int = 1,
                             pixel_shuffle: bool = False, use_tile_tags: bool = False) -> int:
    """Embeddings one image tile contributes to the language model's sequence."""
    n = (img_h // patch_dim) * (img_w // patch_dim)
    keep_class = vision_model_type in ("clip", "radio", "internvit") and not disable_vision_class_token
    if vision_model_type == "siglip":
        keep_class = False
    if keep_class:
        n += class_token_len
    if pixel_shuffle:
        n = int((n - (class_token_len if keep_class else 0)) * 0.25) + (class_token_len if keep_class else 0)
    if use_tile_tags:
        n += 5
    return n


class _PatchEmbed(nn.Module):
    def __init__(self, config, patch_dim, bias):
        super().__init__()
        self.patch_dim = patch_dim
        self.proj = nn.Linear(3 * patch_dim * patch_dim, config.hidden_size, bias=bias, device=_device(config),
                              dtype=config.params_dtype)

    def forward(self, x):
        p = self.patch_dim
        patches = F.unfold(x, kernel_size=p, stride=p).transpose(1, 2)        # [b, n, 3*p*p]
        return self.proj(patches.to(self.proj.weight.dtype))


class CLIPViTModel(nn.Module):
    def __init__(self, transformer_config: TransformerConfig, transformer_layer_spec=None, ln_pre_impl=None,
                 ln_post_impl=None, add_class_token: bool = True, class_token_len: int = 1, patch_dim: int = 14,
                 img_h: int = 336, img_w: int = 336, model_subtype: str = "clip"):
        super().__init__()
        cfg = self.config = transformer_config
        self.patch_dim, self.img_h, self.img_w = patch_dim, img_h, img_w
        self.class_token_len = class_token_len if add_class_token else 0
        self.num_patches = (img_h // patch_dim) * (img_w // patch_dim)
        self.seq_length = self.num_patches + self.class_token_len
        self.subtype = model_subtype
        conv_bias = model_subtype in ("siglip", "internvit")
        self.conv1 = _PatchEmbed(cfg, patch_dim, conv_bias)
        self.position_embeddings = nn.Embedding(self.seq_length, cfg.hidden_size, device=_device(cfg),
                                                dtype=cfg.params_dtype)
        if add_class_token:
            self.class_token = nn.Parameter(torch.randn(1, self.class_token_len, cfg.hidden_size, device=_device(cfg),
                                                        dtype=cfg.params_dtype))
        else:
            self.register_parameter("class_token", None)
        self.ln_pre = Norm(cfg, cfg.hidden_size) if model_subtype == "clip" else None
        self.decoder = TransformerBlock(cfg, True, True, causal=False, post_layer_norm=model_subtype == "siglip")
        self.ln_post = None

    def set_input_tensor(self, t):
        self.decoder.set_input_tensor(t)

    def forward(self, x: torch.Tensor, attention_mask: Optional[torch.Tensor] = None):
        h = self.conv1(x)                                                     # [b, n, hid]
        if self.class_token is not None:
            h = torch.cat((self.class_token.expand(h.shape[0], -1, -1), h), dim=1)
        h = h + self.position_embeddings.weight[: h.shape[1]].unsqueeze(0)
        if self.ln_pre is not None:
            h = self.ln_pre(h)
        h = self.decoder(h.transpose(0, 1).contiguous(), attention_mask=attention_mask)
        return h.transpose(0, 1).contiguous()                                 # [b, s, hid]


class RADIOViTModel(CLIPViTModel):
    """RADIO backbone: several class ("summary") tokens, bias in the patch embedding, interpolated
    position table for other resolutions, no pre-norm."""

    def __init__(self, transformer_config, transformer_layer_spec=None, add_class_token=True, class_token_len=8,
                 patch_dim=16, img_h=224, img_w=224, max_img_h=2048, max_img_w=2048, pos_dropout=0.0, **kw):
        super().__init__(transformer_config, add_class_token=add_class_token, class_token_len=class_token_len,
                         patch_dim=patch_dim, img_h=img_h, img_w=img_w, model_subtype="radio")
        cfg = transformer_config
        self.conv1 = _PatchEmbed(cfg, patch_dim, True)
        self.max_grid = (max_img_h // patch_dim, max_img_w // patch_dim)
        self.position_embeddings = None
        self.pos_table = nn.Parameter(torch.randn(1, self.max_grid[0] * self.max_grid[1], cfg.hidden_size,
                                                  device=_device(cfg), dtype=cfg.params_dtype) * 0.02)

    def _pos(self, gh, gw):
        t = self.pos_table.view(1, self.max_grid[0], self.max_grid[1], -1).permute(0, 3, 1, 2).float()
        t = F.interpolate(t, size=(gh, gw), mode="bilinear", align_corners=False)
        return t.permute(0, 2, 3, 1).reshape(1, gh * gw, -1).to(self.pos_table.dtype)

    def forward(self, x, attention_mask=None):
        gh, gw = x.shape[2] // self.patch_dim, x.shape[3] // self.patch_dim
        h = self.conv1(x) + self._pos(gh, gw)
        if self.class_token is not None:
            h = torch.cat((self.class_token.expand(h.shape[0], -1, -1), h), dim=1)
        h = self.decoder(h.transpose(0, 1).contiguous(), attention_mask=attention_mask)
        return h.transpose(0, 1).contiguous()


class MultimodalProjector(nn.Module):
    """'mlp' (two tensor-parallel linears with the config's activation) or 'affine' (one linear)."""

    def __init__(self, config: TransformerConfig, submodules=None, projector_type: str = "mlp", input_size: int = 0):
        super().__init__()
        self.projector_type = projector_type
        if projector_type == "mlp":
            self.linear_fc1 = ColumnParallelLinear(input_size, config.ffn_hidden_size, config=config,
                                                   init_method=config.init_method, bias=config.add_bias_linear,
                                                   skip_bias_add=False)
            self.linear_fc2 = RowParallelLinear(config.ffn_hidden_size, config.hidden_size, config=config,
                                                init_method=config.output_layer_init_method,
                                                bias=config.add_bias_linear, skip_bias_add=False)
        elif projector_type == "affine":
            self.linear = ColumnParallelLinear(input_size, config.hidden_size, config=config,
                                               init_method=config.init_method, bias=config.add_bias_linear,
                                               gather_output=True)
        else:
            raise ValueError(f"unknown projector type {projector_type}")

    def forward(self, h):
        if self.projector_type == "affine":
            return self.linear(h)[0]
        x, _ = self.linear_fc1(h)
        x = F.gelu(x)
        return self.linear_fc2(x)[0]


class VitClassificationModel(nn.Module):
    """ViT backbone + linear head on the class token: image [b, c, h, w] -> logits [b, num_classes]
    (reference: megatron/legacy/model/vision/classification.py:15, the model of pretrain_vision_classify.py)."""

    def __init__(self, config: TransformerConfig, num_classes: int, img_h: int = 224, img_w: int = 224,
                 patch_dim: int = 16, pre_process: bool = True, post_process: bool = True):
        super().__init__()
        self.config = config
        self.backbone = CLIPViTModel(config, patch_dim=patch_dim, img_h=img_h, img_w=img_w, add_class_token=True)
        self.head = nn.Linear(config.hidden_size, num_classes, device=_device(config), dtype=config.params_dtype)
        nn.init.zeros_(self.head.weight)
        nn.init.zeros_(self.head.bias)

    def set_input_tensor(self, t):
        self.backbone.set_input_tensor(t)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        h = self.backbone(images)                           # [b, 1 + patches, hidden]
        return self.head(h[:, 0])
