"""Vision transformers and the projector that feeds them to a language model.

Reference: megatron/core/models/vision/clip_vit_model.py (``CLIPViTModel`` :26,
``get_num_image_embeddings`` :224), vision/radio.py (``RADIOViTModel`` :29),
vision/multimodal_projector.py (``MultimodalProjector`` :18), vision/vit_layer_specs.py.
Images [b, 3, H, W] are cut into patches and embedded by one GEMM (the strided conv of the reference is
a linear map on the unfolded patches), prefixed with class tokens, given learned positions and run
through a bidirectional transformer block.
"""
from __future__ import annotations

import math
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

    def _interpolated_positions(self, gh: int, gw: int) -> torch.Tensor:
        """Position table for an image of another size (multi-crop training): the patch part is resized
        bicubically on its grid, the class-token rows are kept."""
        w = self.position_embeddings.weight
        k = self.class_token_len
        g0h, g0w = self.img_h // self.patch_dim, self.img_w // self.patch_dim
        grid = w[k:].view(1, g0h, g0w, -1).permute(0, 3, 1, 2).float()
        grid = F.interpolate(grid, size=(gh, gw), mode="bicubic", align_corners=False)
        grid = grid.permute(0, 2, 3, 1).reshape(gh * gw, -1).to(w.dtype)
        return torch.cat((w[:k], grid), dim=0).unsqueeze(0)

    def forward(self, x: torch.Tensor, attention_mask: Optional[torch.Tensor] = None):
        h = self.conv1(x)                                                     # [b, n, hid]
        if self.class_token is not None:
            h = torch.cat((self.class_token.expand(h.shape[0], -1, -1), h), dim=1)
        if h.shape[1] == self.seq_length:
            h = h + self.position_embeddings.weight.unsqueeze(0)
        else:
            h = h + self._interpolated_positions(x.shape[2] // self.patch_dim, x.shape[3] // self.patch_dim)
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


# ---------------------------------------------------------------------------------------------- self-supervised ViT
class DINOHead(nn.Module):
    """Projection head of DINO: MLP -> bottleneck -> L2 normalise -> weight-normalised linear to ``out_dim`` prototypes
    (reference: megatron/legacy/model/vision/dino.py:80-125)."""

    def __init__(self, in_dim: int, out_dim: int, hidden_dim: int = 2048, bottleneck_dim: int = 256, nlayers: int = 3,
                 norm_last_layer: bool = True, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        if nlayers <= 1:
            layers = [nn.Linear(in_dim, bottleneck_dim, **kw)]
        else:
            layers = [nn.Linear(in_dim, hidden_dim, **kw), nn.GELU()]
            for _ in range(nlayers - 2):
                layers += [nn.Linear(hidden_dim, hidden_dim, **kw), nn.GELU()]
            layers.append(nn.Linear(hidden_dim, bottleneck_dim, **kw))
        self.mlp = nn.Sequential(*layers)
        for m in self.mlp:
            if isinstance(m, nn.Linear):
                nn.init.trunc_normal_(m.weight, std=0.02)
                nn.init.zeros_(m.bias)
        # weight normalisation written out: direction v (trained), gain g (fixed at one with norm_last_layer)
        self.last_v = nn.Parameter(torch.empty(out_dim, bottleneck_dim, **kw))
        nn.init.trunc_normal_(self.last_v, std=0.02)
        self.last_g = nn.Parameter(torch.ones(out_dim, 1, **kw), requires_grad=not norm_last_layer)

        self.freeze_last = False

    def forward(self, x):
        x = F.normalize(self.mlp(x), dim=-1, p=2)
        v = self.last_v
        if self.freeze_last and v.requires_grad and torch.is_grad_enabled():
            # the gradient still arrives (gradient-buffer accounting stays whole) but as zeros
            v = v * 1.0
            v.register_hook(torch.zeros_like)
        w = self.last_g * F.normalize(v, dim=1)
        return F.linear(x, w)


class DINOLoss(nn.Module):
    """Cross entropy between the teacher's centred, sharpened distribution of a global view and the student's
    distribution of every other view; the centre is an exponential moving average of the teacher outputs over the
    data-parallel group (reference: dino.py:128-195)."""

    def __init__(self, out_dim: int, ncrops: int, warmup_teacher_temp: float, teacher_temp: float,
                 warmup_teacher_temp_iters: int, total_iters: int, student_temp: float = 0.1,
                 center_momentum: float = 0.9, group=None):
        super().__init__()
        self.student_temp, self.center_momentum, self.ncrops, self.group = student_temp, center_momentum, ncrops, group
        self.register_buffer("center", torch.zeros(1, out_dim))
        warm = max(min(warmup_teacher_temp_iters, total_iters), 0)
        self.temps = torch.cat((torch.linspace(warmup_teacher_temp, teacher_temp, warm) if warm else torch.zeros(0),
                                torch.full((max(total_iters - warm, 1),), teacher_temp)))

    def teacher_temp(self, iteration: int) -> float:
        return float(self.temps[min(iteration, len(self.temps) - 1)])

    def forward(self, student_output: torch.Tensor, teacher_output: torch.Tensor, iteration: int) -> torch.Tensor:
        s = (student_output.float() / self.student_temp).chunk(self.ncrops)
        t = F.softmax((teacher_output.float() - self.center) / self.teacher_temp(iteration), dim=-1).detach().chunk(2)
        total, terms = 0.0, 0
        for iq, q in enumerate(t):
            for v in range(len(s)):
                if v == iq:
                    continue                                  # a view is never compared with itself
                total = total + torch.sum(-q * F.log_softmax(s[v], dim=-1), dim=-1).mean()
                terms += 1
        self.update_center(teacher_output)
        return total / terms

    @torch.no_grad()
    def update_center(self, teacher_output: torch.Tensor):
        batch = teacher_output.float().sum(dim=0, keepdim=True)
        count = torch.tensor([float(teacher_output.shape[0])], device=batch.device)
        if self.group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(self.group) > 1:
            torch.distributed.all_reduce(batch, group=self.group)
            torch.distributed.all_reduce(count, group=self.group)
        self.center.mul_(self.center_momentum).add_((batch / count) * (1 - self.center_momentum))


def cosine_schedule(base: float, final: float, total_iters: int) -> torch.Tensor:
    it = torch.arange(max(total_iters, 1), dtype=torch.float32)
    return final + 0.5 * (base - final) * (1 + torch.cos(math.pi * it / max(total_iters, 1)))


class DINOPretrainModel(nn.Module):
    """Student and momentum teacher (a backbone - ViT, or MiT / Swin with ``backbone_type`` - + ``DINOHead`` each).  Training: ``forward(list of crops)`` runs the
    student over all crops (one backbone pass per resolution) and the teacher over the two global crops, and returns
    (student output, teacher output); evaluation returns the teacher's class-token features for the k-NN monitor.
    ``after_optimizer_step`` moves the teacher towards the student with a momentum that follows a cosine from 0.996
    to 1 (reference: dino.py:217-292, ``update_momentum``, ``cancel_gradients_last_layer``)."""

    def __init__(self, config: TransformerConfig, *, img_h: int = 224, img_w: int = 224, patch_dim: int = 16,
                 out_dim: int = 65536, head_hidden: int = 2048, bottleneck: int = 256, norm_last_layer: bool = False,
                 local_crops: int = 10, warmup_teacher_temp: float = 0.04, teacher_temp: float = 0.07,
                 warmup_teacher_temp_iters: int = 0, total_iters: int = 1, freeze_last_layer_iters: int = 0,
                 base_momentum: float = 0.996, dp_group=None, backbone_type: str = "vit", swin_type: str = "tiny"):
        super().__init__()
        self.config = config
        self.backbone_type = backbone_type
        dev, dt = _device(config), config.params_dtype

        def tower(norm_last, teacher):
            if backbone_type == "vit":
                backbone, width = CLIPViTModel(config, patch_dim=patch_dim, img_h=img_h, img_w=img_w,
                                               add_class_token=True), config.hidden_size
            else:       # hierarchical backbones return the pooled feature vector themselves
                from .vision_backbones import build_feature_backbone
                backbone, width = build_feature_backbone(backbone_type, config, img_h=img_h, img_w=img_w,
                                                         patch_dim=patch_dim, swin_type=swin_type, teacher=teacher)
            return nn.ModuleDict({
                "backbone": backbone,
                "head": DINOHead(width, out_dim, head_hidden, bottleneck, norm_last_layer=norm_last,
                                 device=dev, dtype=dt)})
        self.student = tower(norm_last_layer, False)
        self.teacher = tower(True, True)
        self.teacher.load_state_dict(self.student.state_dict())
        for p in self.teacher.parameters():
            p.requires_grad_(False)
        # the student's backbone runs once per crop resolution: several partial gradients per parameter and step
        for p in self.student["backbone"].parameters():
            p.expected_grad_signals = 2
        self.dino_loss = DINOLoss(out_dim, local_crops + 2, warmup_teacher_temp, teacher_temp, warmup_teacher_temp_iters,
                                  total_iters, group=dp_group)
        self.momentum = cosine_schedule(base_momentum, 1.0, total_iters)
        self.freeze_last_layer_iters = freeze_last_layer_iters

    def set_input_tensor(self, t):
        pass

    def _features(self, tower, images):
        out = tower["backbone"](images)
        return out[:, 0] if self.backbone_type == "vit" else out

    def forward(self, images):
        if not self.training:
            with torch.no_grad():
                x = images[0] if isinstance(images, (list, tuple)) else images
                return None, self._features(self.teacher, x)
        crops = list(images) if isinstance(images, (list, tuple)) else [images]
        with torch.no_grad():
            t_out = self.teacher["head"](self._features(self.teacher, torch.cat(crops[:2], dim=0)))
        # one backbone pass per run of equal-resolution crops
        feats, start = [], 0
        while start < len(crops):
            end = start
            while end < len(crops) and crops[end].shape[-2:] == crops[start].shape[-2:]:
                end += 1
            feats.append(self._features(self.student, torch.cat(crops[start:end], dim=0)))
            start = end
        return self.student["head"](torch.cat(feats, dim=0)), t_out

    def set_iteration(self, iteration: int):
        """The prototype layer gets zero gradients during the first iterations (stabilises the start of training;
        the reference drops the gradient instead, ``cancel_gradients_last_layer``)."""
        self.student["head"].freeze_last = iteration < self.freeze_last_layer_iters

    @torch.no_grad()
    def after_optimizer_step(self, iteration: int):
        m = float(self.momentum[min(iteration, len(self.momentum) - 1)])
        for ps, pt in zip(self.student.parameters(), self.teacher.parameters()):
            pt.mul_(m).add_(ps.detach().to(pt.dtype), alpha=1 - m)


@torch.no_grad()
def knn_predict(feature: torch.Tensor, feature_bank: torch.Tensor, feature_labels: torch.Tensor, classes: int,
                knn_k: int, knn_t: float) -> torch.Tensor:
    """Weighted k-nearest-neighbour vote: ``feature`` [b, d] against ``feature_bank`` [d, n] (both L2-normalised);
    returns class indices sorted by score, [b, classes] (reference: megatron/legacy/model/vision/knn_monitor.py:96-128)."""
    sim = feature @ feature_bank
    k = min(knn_k, feature_bank.shape[1])
    w, idx = sim.topk(k=k, dim=-1)
    labels = feature_labels.expand(feature.shape[0], -1).gather(-1, idx)
    w = (w / knn_t).exp()
    one_hot = torch.zeros(feature.shape[0] * k, classes, device=feature.device)
    one_hot.scatter_(-1, labels.reshape(-1, 1), 1.0)
    scores = (one_hot.view(feature.shape[0], k, classes) * w.unsqueeze(-1)).sum(dim=1)
    return scores.argsort(dim=-1, descending=True)


class VitInpaintingModel(nn.Module):
    """ViT backbone + linear decoder from every patch token to its pixels: masked image [b, 3, h, w] -> reconstruction
    of the same shape (reference: megatron/legacy/model/vision/inpainting.py:20-66)."""

    def __init__(self, config: TransformerConfig, img_h: int = 224, img_w: int = 224, patch_dim: int = 16):
        super().__init__()
        self.config, self.patch_dim, self.img_h, self.img_w = config, patch_dim, img_h, img_w
        self.backbone = CLIPViTModel(config, patch_dim=patch_dim, img_h=img_h, img_w=img_w, add_class_token=True)
        self.linear_decoder = nn.Linear(config.hidden_size, 3 * patch_dim * patch_dim, device=_device(config),
                                        dtype=config.params_dtype)
        nn.init.trunc_normal_(self.linear_decoder.weight, std=0.02)
        nn.init.zeros_(self.linear_decoder.bias)

    def set_input_tensor(self, t):
        self.backbone.set_input_tensor(t)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        h = self.backbone(images)[:, self.backbone.class_token_len:]          # [b, patches, hidden]
        px = self.linear_decoder(h).transpose(1, 2)                           # [b, 3*p*p, patches]
        return F.fold(px.float(), output_size=images.shape[-2:], kernel_size=self.patch_dim, stride=self.patch_dim)


def random_patch_mask(b: int, img_h: int, img_w: int, patch_dim: int, mask_factor: float = 1.0, mask_type: str = "random",
                      generator=None) -> torch.Tensor:
    """1 where the image is hidden.  ``random``: a random walk over the patch grid that covers about
    ``mask_factor`` x a quarter of the patches; ``row``: a band of whole patch rows of that area."""
    gh, gw = img_h // patch_dim, img_w // patch_dim
    target = max(1, min(gh * gw - 1, int(round(mask_factor * gh * gw / 4))))
    mask = torch.zeros(b, gh, gw)
    for i in range(b):
        if mask_type == "row":
            rows = max(1, min(gh - 1, int(round(target / gw))))
            r0 = int(torch.randint(0, gh - rows + 1, (1,), generator=generator))
            mask[i, r0:r0 + rows] = 1
            continue
        y, x = int(torch.randint(0, gh, (1,), generator=generator)), int(torch.randint(0, gw, (1,), generator=generator))
        covered = 0
        while covered < target:
            if mask[i, y, x] == 0:
                mask[i, y, x] = 1
                covered += 1
            step = int(torch.randint(0, 4, (1,), generator=generator))
            y = min(max(y + (step == 0) - (step == 1), 0), gh - 1)
            x = min(max(x + (step == 2) - (step == 3), 0), gw - 1)
    return mask.repeat_interleave(patch_dim, 1).repeat_interleave(patch_dim, 2).unsqueeze(1)


def psnr(pred: torch.Tensor, target: torch.Tensor, max_val: float = 1.0) -> torch.Tensor:
    mse = (pred.float() - target.float()).pow(2).flatten(1).mean(dim=1).clamp(min=1e-12)
    return (10.0 * torch.log10(max_val ** 2 / mse)).mean()


def ssim(pred: torch.Tensor, target: torch.Tensor, window: int = 11, max_val: float = 1.0) -> torch.Tensor:
    """Structural similarity with a Gaussian window (sigma 1.5), averaged over channels and positions."""
    x, y = pred.float(), target.float()
    c = x.shape[1]
    ax = torch.arange(window, dtype=torch.float32, device=x.device) - window // 2
    g = torch.exp(-ax.pow(2) / (2 * 1.5 ** 2))
    g = (g / g.sum()).unsqueeze(0)
    k = (g.t() @ g).expand(c, 1, window, window).contiguous()
    mu_x, mu_y = F.conv2d(x, k, groups=c), F.conv2d(y, k, groups=c)
    sxx = F.conv2d(x * x, k, groups=c) - mu_x ** 2
    syy = F.conv2d(y * y, k, groups=c) - mu_y ** 2
    sxy = F.conv2d(x * y, k, groups=c) - mu_x * mu_y
    c1, c2 = (0.01 * max_val) ** 2, (0.03 * max_val) ** 2
    return (((2 * mu_x * mu_y + c1) * (2 * sxy + c2)) / ((mu_x ** 2 + mu_y ** 2 + c1) * (sxx + syy + c2))).mean()
