"""Hierarchical vision backbones beside the plain ViT: Mix Transformer (MiT, the SegFormer encoder) and Swin.

Reference: megatron/legacy/model/vision/mit_backbone.py (``MixVisionTransformer`` :204, presets ``mit_b0`` .. ``mit_b5``
:357-415), esvit_swin_backbone.py / swin_backbone.py (``SwinTransformer``, ``get_swin`` :810 / :605),
classification.py:58 (``MitClassificationModel``), inpainting.py:84 (``MitInpaintingModel``) and dino.py:179-215
(backbone choice of the student and teacher).

Both backbones are four stages of transformer blocks over a feature map that halves in resolution and widens from
stage to stage.  MiT embeds overlapping patches with a strided convolution, lets every query attend to a spatially
reduced copy of the map, and puts a depth-wise 3 x 3 convolution inside its feed-forward block (which is what gives it
positions).  Swin attends inside non-overlapping windows that are shifted by half a window in every second block, with
a learned bias per relative offset, and merges 2 x 2 neighbours between stages.  These models are data parallel only
(no tensor-parallel shards), as in the reference.

The blocks are written with PyTorch operators, as the reference's are.  ``USE_FUSED_KERNELS = True`` sends the layer
norms to the framework's fused kernel and MiT's attention (head size 64, no bias term) to its flash kernel; that path
is off by default because it has not passed a comparison on a GPU yet (MiT's first stage attends to as few as four
keys, far below the key tile the flash kernel was tested with).  Swin's windowed attention carries an additive bias
and is always computed with plain matrix products.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops.attention import attention as flash_attention

# True: layer norms and MiT's attention on the framework's own kernels when the tensors are on a GPU.
USE_FUSED_KERNELS = False


class _LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))

    def forward(self, x):
        if USE_FUSED_KERNELS and x.is_cuda and x.shape[-1] % 8 == 0:
            return ops.layernorm(x.contiguous(), self.weight, self.bias, self.eps)
        return F.layer_norm(x, x.shape[-1:], self.weight, self.bias, self.eps)


class DropPath(nn.Module):
    """Stochastic depth: drops the whole residual branch of a sample with probability ``p`` while training."""

    def __init__(self, p: float = 0.0):
        super().__init__()
        self.p = float(p)

    def forward(self, x):
        if self.p == 0.0 or not self.training:
            return x
        keep = 1.0 - self.p
        mask = torch.rand(x.shape[0], *([1] * (x.dim() - 1)), device=x.device, dtype=torch.float32) < keep
        return x * (mask.to(x.dtype) / keep)


def _init_weights(m: nn.Module):
    if isinstance(m, nn.Linear):
        nn.init.trunc_normal_(m.weight, std=0.02)
        if m.bias is not None:
            nn.init.zeros_(m.bias)
    elif isinstance(m, nn.Conv2d):
        fan_out = m.kernel_size[0] * m.kernel_size[1] * m.out_channels // m.groups
        nn.init.normal_(m.weight, 0.0, math.sqrt(2.0 / fan_out))
        if m.bias is not None:
            nn.init.zeros_(m.bias)


def _attend(q, k, v, bias=None):
    """q [b, heads, nq, d], k / v [b, heads, nk, d], optional additive ``bias`` broadcastable to [b, heads, nq, nk]."""
    d = q.shape[-1]
    if (USE_FUSED_KERNELS and bias is None and q.is_cuda and d in (64, 128)
            and q.dtype in (torch.bfloat16, torch.float16)):
        # the flash kernel's layout: q [sq, b, groups, 1, d], k / v [sk, b, groups, d]
        o = flash_attention(q.permute(2, 0, 1, 3).unsqueeze(3), k.permute(2, 0, 1, 3), v.permute(2, 0, 1, 3), causal=False)
        return o.permute(1, 2, 0, 3)                                            # [b, heads, nq, d]
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) / math.sqrt(d)
    if bias is not None:
        s = s + bias.float()
    return torch.matmul(torch.softmax(s, dim=-1).to(v.dtype), v)


# ------------------------------------------------------------------------------------------------ Mix Transformer
class _ReducedAttention(nn.Module):
    """Self-attention whose keys and values come from the map reduced ``sr`` times in each direction."""

    def __init__(self, dim, heads, sr, qkv_bias, kw):
        super().__init__()
        self.heads, self.sr = heads, sr
        self.q = nn.Linear(dim, dim, bias=qkv_bias, **kw)
        self.kv = nn.Linear(dim, 2 * dim, bias=qkv_bias, **kw)
        self.proj = nn.Linear(dim, dim, **kw)
        if sr > 1:
            self.reduce = nn.Conv2d(dim, dim, kernel_size=sr, stride=sr, **kw)
            self.reduce_norm = _LayerNorm(dim, 1e-5, **kw)

    def forward(self, x, hw):
        b, n, c = x.shape
        q = self.q(x).view(b, n, self.heads, c // self.heads).transpose(1, 2)
        if self.sr > 1:
            m = self.reduce(x.transpose(1, 2).reshape(b, c, *hw)).flatten(2).transpose(1, 2)
            m = self.reduce_norm(m)
        else:
            m = x
        kv = self.kv(m).view(b, m.shape[1], 2, self.heads, c // self.heads).permute(2, 0, 3, 1, 4)
        o = _attend(q, kv[0], kv[1]).transpose(1, 2).reshape(b, n, c)
        return self.proj(o)


class _MixFFN(nn.Module):
    """Linear -> depth-wise 3 x 3 convolution over the map -> GELU -> linear."""

    def __init__(self, dim, hidden, kw):
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden, **kw)
        self.dwconv = nn.Conv2d(hidden, hidden, 3, 1, 1, groups=hidden, **kw)
        self.fc2 = nn.Linear(hidden, dim, **kw)

    def forward(self, x, hw):
        b, n, _ = x.shape
        h = self.fc1(x)
        h = self.dwconv(h.transpose(1, 2).reshape(b, -1, *hw)).flatten(2).transpose(1, 2)
        return self.fc2(F.gelu(h))


class _MitBlock(nn.Module):
    def __init__(self, dim, heads, mlp_ratio, sr, qkv_bias, drop_path, kw):
        super().__init__()
        self.norm1 = _LayerNorm(dim, **kw)
        self.attn = _ReducedAttention(dim, heads, sr, qkv_bias, kw)
        self.norm2 = _LayerNorm(dim, **kw)
        self.mlp = _MixFFN(dim, int(dim * mlp_ratio), kw)
        self.drop_path = DropPath(drop_path)

    def forward(self, x, hw):
        x = x + self.drop_path(self.attn(self.norm1(x), hw))
        return x + self.drop_path(self.mlp(self.norm2(x), hw))


class _MitStage(nn.Module):
    def __init__(self, in_ch, dim, depth, heads, mlp_ratio, sr, patch, stride, qkv_bias, drop_paths, kw):
        super().__init__()
        self.embed = nn.Conv2d(in_ch, dim, kernel_size=patch, stride=stride, padding=patch // 2, **kw)
        self.embed_norm = _LayerNorm(dim, 1e-5, **kw)
        self.blocks = nn.ModuleList(_MitBlock(dim, heads, mlp_ratio, sr, qkv_bias, dp, kw) for dp in drop_paths)
        self.norm = _LayerNorm(dim, **kw)

    def forward(self, x):
        x = self.embed(x)
        hw = x.shape[-2:]
        x = self.embed_norm(x.flatten(2).transpose(1, 2))
        for blk in self.blocks:
            x = blk(x, hw)
        return self.norm(x), hw                                                 # tokens [b, h*w, dim]


MIT_PRESETS = {
    # name: (widths, heads, depths)
    "b0": ((32, 64, 160, 256), (1, 2, 5, 8), (2, 2, 2, 2)),
    "b1": ((64, 128, 320, 512), (1, 2, 5, 8), (2, 2, 2, 2)),
    "b2": ((64, 128, 320, 512), (1, 2, 5, 8), (3, 4, 6, 3)),
    "b3": ((64, 128, 320, 512), (1, 2, 5, 8), (3, 4, 18, 3)),
    "b4": ((64, 128, 320, 512), (1, 2, 5, 8), (3, 8, 27, 3)),
    "b5": ((64, 128, 320, 512), (1, 2, 5, 8), (3, 6, 40, 3)),
}


class MixVisionTransformer(nn.Module):
    """Image [b, c, H, W] -> the four feature maps [b, width_i, H / 4 / 2^i, W / 4 / 2^i], or with ``output_avg`` the
    mean of the last stage's tokens [b, width_3]."""

    def __init__(self, widths: Sequence[int] = (64, 128, 320, 512), heads: Sequence[int] = (1, 2, 5, 8),
                 depths: Sequence[int] = (3, 4, 6, 3), mlp_ratios: Sequence[float] = (4, 4, 4, 4),
                 sr_ratios: Sequence[int] = (8, 4, 2, 1), in_chans: int = 3, qkv_bias: bool = True,
                 drop_path_rate: float = 0.1, output_avg: bool = False, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.widths, self.output_avg = tuple(widths), output_avg
        self.num_features = widths[-1]
        rates = torch.linspace(0, drop_path_rate, sum(depths)).tolist()
        self.stages = nn.ModuleList()
        at, prev = 0, in_chans
        for i in range(4):
            self.stages.append(_MitStage(prev, widths[i], depths[i], heads[i], mlp_ratios[i], sr_ratios[i],
                                         7 if i == 0 else 3, 4 if i == 0 else 2, qkv_bias,
                                         rates[at:at + depths[i]], kw))
            at, prev = at + depths[i], widths[i]
        self.apply(_init_weights)

    @classmethod
    def preset(cls, name: str, **kwargs) -> "MixVisionTransformer":
        widths, heads, depths = MIT_PRESETS[name]
        return cls(widths=widths, heads=heads, depths=depths, **kwargs)

    def forward(self, x):
        maps: List[torch.Tensor] = []
        x = x.to(self.stages[0].embed.weight.dtype)
        for i, stage in enumerate(self.stages):
            tokens, hw = stage(x)
            if i == 3 and self.output_avg:
                return tokens.mean(dim=1)
            x = tokens.transpose(1, 2).reshape(tokens.shape[0], -1, *hw)
            maps.append(x)
        return maps


# ------------------------------------------------------------------------------------------------------------ Swin
class _WindowAttention(nn.Module):
    """Attention among the tokens of one window with a learned bias per relative offset; the table covers offsets of
    a full ``window`` and a smaller window (a map smaller than the window) reads its centre."""

    def __init__(self, dim, heads, window, qkv_bias, kw):
        super().__init__()
        self.heads, self.window = heads, window
        self.qkv = nn.Linear(dim, 3 * dim, bias=qkv_bias, **kw)
        self.proj = nn.Linear(dim, dim, **kw)
        self.bias_table = nn.Parameter(torch.zeros((2 * window - 1) ** 2, heads, **kw))
        nn.init.trunc_normal_(self.bias_table, std=0.02)
        self._index = {}

    def _relative_index(self, ws: int, device) -> torch.Tensor:
        key = (ws, str(device))
        if key not in self._index:
            r = torch.arange(ws, device=device)
            yy, xx = torch.meshgrid(r, r, indexing="ij")
            pts = torch.stack([yy.flatten(), xx.flatten()])                       # [2, ws*ws]
            rel = pts[:, :, None] - pts[:, None, :] + (self.window - 1)             # offsets in 0 .. 2*window-2
            self._index[key] = (rel[0] * (2 * self.window - 1) + rel[1]).flatten()
        return self._index[key]

    def forward(self, x, ws: int, mask: Optional[torch.Tensor]):
        nb, n, c = x.shape                                                       # nb = batch * windows
        qkv = self.qkv(x).view(nb, n, 3, self.heads, c // self.heads).permute(2, 0, 3, 1, 4)
        bias = self.bias_table[self._relative_index(ws, x.device)].view(n, n, self.heads).permute(2, 0, 1)[None]
        if mask is not None:                                                     # [windows, n, n]
            nw = mask.shape[0]
            bias = (bias + mask[:, None]).repeat(nb // nw, 1, 1, 1)
        o = _attend(qkv[0], qkv[1], qkv[2], bias).transpose(1, 2).reshape(nb, n, c)
        return self.proj(o)


def _windows(x, ws):
    """[b, H, W, c] -> [b * windows, ws*ws, c]."""
    b, h, w, c = x.shape
    return x.view(b, h // ws, ws, w // ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(-1, ws * ws, c)


def _unwindows(x, ws, b, h, w):
    c = x.shape[-1]
    return x.view(b, h // ws, w // ws, ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(b, h, w, c)


class _SwinBlock(nn.Module):
    def __init__(self, dim, heads, window, shifted, mlp_ratio, qkv_bias, drop_path, kw):
        super().__init__()
        self.window, self.shifted = window, shifted
        self.norm1 = _LayerNorm(dim, **kw)
        self.attn = _WindowAttention(dim, heads, window, qkv_bias, kw)
        self.norm2 = _LayerNorm(dim, **kw)
        self.fc1 = nn.Linear(dim, int(dim * mlp_ratio), **kw)
        self.fc2 = nn.Linear(int(dim * mlp_ratio), dim, **kw)
        self.drop_path = DropPath(drop_path)
        self._masks = {}

    def _shift_mask(self, hp, wp, ws, shift, device):
        """Tokens that the cyclic shift brought together from opposite borders must not attend to each other."""
        key = (hp, wp, ws, shift, str(device))
        if key not in self._masks:
            region = torch.zeros(1, hp, wp, 1, device=device)
            cuts = (slice(0, -ws), slice(-ws, -shift), slice(-shift, None))
            n = 0
            for ys in cuts:
                for xs in cuts:
                    region[:, ys, xs] = n
                    n += 1
            ids = _windows(region, ws).squeeze(-1)                                # [windows, ws*ws]
            self._masks[key] = (ids[:, None, :] != ids[:, :, None]).float() * -100.0
        return self._masks[key]

    def forward(self, x, hw):
        h, w = hw
        b, n, c = x.shape
        ws = min(self.window, h, w)
        shift = self.window // 2 if (self.shifted and min(h, w) > self.window) else 0
        y = self.norm1(x).view(b, h, w, c)
        pad_h, pad_w = (-h) % ws, (-w) % ws
        if pad_h or pad_w:
            y = F.pad(y, (0, 0, 0, pad_w, 0, pad_h))
        hp, wp = h + pad_h, w + pad_w
        mask = None
        if shift:
            y = torch.roll(y, shifts=(-shift, -shift), dims=(1, 2))
            mask = self._shift_mask(hp, wp, ws, shift, x.device)
        y = _unwindows(self.attn(_windows(y, ws), ws, mask), ws, b, hp, wp)
        if shift:
            y = torch.roll(y, shifts=(shift, shift), dims=(1, 2))
        y = y[:, :h, :w].reshape(b, n, c)
        x = x + self.drop_path(y)
        return x + self.drop_path(self.fc2(F.gelu(self.fc1(self.norm2(x)))))


class _PatchMerging(nn.Module):
    """2 x 2 neighbours side by side in the channel dimension, normalised and projected to twice the width."""

    def __init__(self, dim, kw):
        super().__init__()
        self.norm = _LayerNorm(4 * dim, **kw)
        self.reduction = nn.Linear(4 * dim, 2 * dim, bias=False, **kw)

    def forward(self, x, hw):
        h, w = hw
        b, _, c = x.shape
        x = x.view(b, h, w, c)
        if h % 2 or w % 2:
            x = F.pad(x, (0, 0, 0, w % 2, 0, h % 2))
        x = torch.cat([x[:, 0::2, 0::2], x[:, 1::2, 0::2], x[:, 0::2, 1::2], x[:, 1::2, 1::2]], dim=-1)
        hw = (x.shape[1], x.shape[2])
        return self.reduction(self.norm(x.view(b, -1, 4 * c))), hw


SWIN_PRESETS = {
    # name: (width, depths, heads, drop path)
    "tiny": (96, (2, 2, 6, 2), (3, 6, 12, 24), 0.1),
    "base": (128, (2, 2, 18, 2), (4, 8, 16, 32), 0.2),
    "h3": (384, (2, 2, 18, 2), (6, 12, 24, 48), 0.2),
}


class SwinTransformer(nn.Module):
    """Image [b, c, H, W] -> mean of the last stage's tokens [b, 8 * width] (``output_avg``, the default) or those
    tokens as a map [b, 8 * width, H / 32, W / 32]."""

    def __init__(self, width: int = 96, depths: Sequence[int] = (2, 2, 6, 2), heads: Sequence[int] = (3, 6, 12, 24),
                 window: int = 7, patch: int = 4, in_chans: int = 3, mlp_ratio: float = 4.0, qkv_bias: bool = True,
                 drop_path_rate: float = 0.1, output_avg: bool = True, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.output_avg = output_avg
        self.num_features = width * 2 ** (len(depths) - 1)
        self.embed = nn.Conv2d(in_chans, width, kernel_size=patch, stride=patch, **kw)
        self.embed_norm = _LayerNorm(width, **kw)
        rates = torch.linspace(0, drop_path_rate, sum(depths)).tolist()
        self.blocks, self.merges = nn.ModuleList(), nn.ModuleList()
        at = 0
        for i, depth in enumerate(depths):
            dim = width * 2 ** i
            self.blocks.append(nn.ModuleList(
                _SwinBlock(dim, heads[i], window, bool(j % 2), mlp_ratio, qkv_bias, rates[at + j], kw)
                for j in range(depth)))
            at += depth
            if i + 1 < len(depths):
                self.merges.append(_PatchMerging(dim, kw))
        self.norm = _LayerNorm(self.num_features, **kw)
        self.apply(_init_weights)

    @classmethod
    def preset(cls, name: str, teacher: bool = False, **kwargs) -> "SwinTransformer":
        width, depths, heads, drop = SWIN_PRESETS[name]
        return cls(width=width, depths=depths, heads=heads, drop_path_rate=0.0 if teacher else drop, **kwargs)

    def forward(self, x):
        x = self.embed(x.to(self.embed.weight.dtype))
        hw = (x.shape[-2], x.shape[-1])
        x = self.embed_norm(x.flatten(2).transpose(1, 2))
        for i, blocks in enumerate(self.blocks):
            for blk in blocks:
                x = blk(x, hw)
            if i < len(self.merges):
                x, hw = self.merges[i](x, hw)
        x = self.norm(x)
        if self.output_avg:
            return x.mean(dim=1)
        return x.transpose(1, 2).reshape(x.shape[0], -1, *hw)


# ------------------------------------------------------------------------------------------------- models on top
def build_feature_backbone(kind: str, config, *, img_h: int = 224, img_w: int = 224, patch_dim: int = 16,
                           swin_type: str = "tiny", teacher: bool = False) -> Tuple[nn.Module, int]:
    """The backbone of a self-supervised tower and the width of its feature vector: ``vit`` (class token of the
    framework's ViT), ``mit`` (MiT-B5, averaged) or ``swin`` (reference: dino.py:179-215).  The teacher's copy has no
    stochastic depth."""
    from ..parallel.layers import _device
    kw = dict(device=_device(config), dtype=config.params_dtype)
    if kind == "vit":
        from .vision import CLIPViTModel

        class _ClassToken(nn.Module):
            def __init__(self):
                super().__init__()
                self.vit = CLIPViTModel(config, patch_dim=patch_dim, img_h=img_h, img_w=img_w, add_class_token=True)

            def forward(self, images):
                return self.vit(images)[:, 0]
        return _ClassToken(), config.hidden_size
    if kind == "mit":
        m = MixVisionTransformer.preset("b5", drop_path_rate=0.0 if teacher else 0.1, output_avg=True, **kw)
        return m, m.num_features
    if kind == "swin":
        m = SwinTransformer.preset(swin_type, teacher=teacher, **kw)
        return m, m.num_features
    raise ValueError(f"unknown vision backbone type {kind!r}")


class MitClassificationModel(nn.Module):
    """MiT-B3 with averaged output + linear head: image -> logits [b, num_classes] (reference:
    classification.py:58-86)."""

    def __init__(self, config, num_classes: int, preset: str = "b3"):
        super().__init__()
        from ..parallel.layers import _device
        kw = dict(device=_device(config), dtype=config.params_dtype)
        self.config = config
        self.backbone = MixVisionTransformer.preset(preset, output_avg=True, **kw)
        self.head = nn.Linear(self.backbone.num_features, num_classes, **kw)
        _init_weights(self.head)

    def set_input_tensor(self, t):
        pass

    def forward(self, images):
        return self.head(self.backbone(images))


class MitInpaintingModel(nn.Module):
    """MiT-B3 + the all-MLP decoder of SegFormer: every stage's map is projected to a common width, brought to the
    first stage's resolution, concatenated and fused by a 1 x 1 convolution; a last 1 x 1 convolution predicts the
    pixels of a ``patch_dim`` x ``patch_dim`` patch per position (reference: inpainting.py:84-152).  The first stage
    works at a quarter of the image's resolution, so ``patch_dim`` is 4."""

    def __init__(self, config, img_h: int = 224, img_w: int = 224, patch_dim: int = 4, preset: str = "b3",
                 embed: int = 768, sync_group=None):
        super().__init__()
        from ..parallel.layers import _device
        if patch_dim != 4:
            raise ValueError("the MiT in-painting decoder predicts 4 x 4 patches (--patch-dim 4)")
        kw = dict(device=_device(config), dtype=config.params_dtype)
        self.config, self.patch_dim, self.img_h, self.img_w = config, patch_dim, img_h, img_w
        self.backbone = MixVisionTransformer.preset(preset, **kw)
        self.project = nn.ModuleList(nn.Linear(w, embed, **kw) for w in self.backbone.widths)
        self.fuse = nn.Conv2d(4 * embed, embed, 1, bias=False, **kw)
        # batch statistics over the whole data-parallel group where one is given (GPU only)
        if sync_group is not None and kw["device"].type == "cuda":
            self.fuse_norm = nn.SyncBatchNorm(embed, process_group=sync_group, **kw)
        else:
            self.fuse_norm = nn.BatchNorm2d(embed, **kw)
        self.dropout = nn.Dropout2d(0.1)
        self.predict = nn.Conv2d(embed, 3 * patch_dim * patch_dim, 1, **kw)
        for m in (*self.project, self.fuse, self.predict):
            _init_weights(m)

    def set_input_tensor(self, t):
        pass

    def forward(self, images):
        maps = self.backbone(images)
        size = maps[0].shape[-2:]
        ups = []
        for m, proj in zip(maps, self.project):
            y = proj(m.flatten(2).transpose(1, 2)).transpose(1, 2).reshape(m.shape[0], -1, *m.shape[-2:])
            ups.append(y if y.shape[-2:] == size else F.interpolate(y, size=size, mode="bilinear", align_corners=False))
        x = self.fuse(torch.cat(ups[::-1], dim=1))
        x = self.dropout(F.relu(self.fuse_norm(x)))
        px = self.predict(x).flatten(2)                                          # [b, 3*p*p, positions]
        return F.fold(px.float(), output_size=images.shape[-2:], kernel_size=self.patch_dim, stride=self.patch_dim)
