"""Self-supervised vision models: DINO head / loss / momentum teacher / k-NN vote, in-painting model, masks, image
metrics, position-table interpolation for other crop sizes (reference: megatron/legacy/model/vision/dino.py,
inpainting.py, knn_monitor.py)."""
import math

import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.vision import (CLIPViTModel, DINOHead, DINOLoss, DINOPretrainModel, VitInpaintingModel,
                                            cosine_schedule, knn_predict, psnr, random_patch_mask, ssim)


def _cfg():
    return TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                             attention_dropout=0.0, use_cpu_initialization=True)


def test_backbone_accepts_other_crop_sizes():
    torch.manual_seed(0)
    vit = CLIPViTModel(_cfg(), patch_dim=8, img_h=32, img_w=32)
    full = vit(torch.randn(2, 3, 32, 32))
    small = vit(torch.randn(2, 3, 16, 16))
    assert full.shape == (2, 17, 32) and small.shape == (2, 5, 32)
    same = vit._interpolated_positions(4, 4)
    assert torch.allclose(same[0], vit.position_embeddings.weight, atol=1e-5)       # identity at the native grid


def test_dino_head_and_loss():
    torch.manual_seed(0)
    head = DINOHead(32, 24, hidden_dim=16, bottleneck_dim=8, norm_last_layer=True)
    assert not head.last_g.requires_grad
    out = head(torch.randn(6, 32))
    assert out.shape == (6, 24)
    w = head.last_g * torch.nn.functional.normalize(head.last_v, dim=1)
    assert torch.allclose(w.norm(dim=1), torch.ones(24), atol=1e-5)
    head.freeze_last = True
    head(torch.randn(6, 32)).sum().backward()
    assert head.last_v.grad is not None and head.last_v.grad.abs().sum() == 0 and head.mlp[0].weight.grad.abs().sum() > 0
    loss = DINOLoss(24, ncrops=4, warmup_teacher_temp=0.04, teacher_temp=0.07, warmup_teacher_temp_iters=4, total_iters=10)
    assert abs(loss.teacher_temp(0) - 0.04) < 1e-6 and abs(loss.teacher_temp(3) - 0.07) < 1e-6 and loss.teacher_temp(99) == loss.teacher_temp(9)
    s, t = torch.randn(4 * 3, 24), torch.randn(2 * 3, 24)
    val = loss(s, t, 0)
    # by hand: teacher view q against every student view v != q
    sv = (s / 0.1).chunk(4)
    tq = torch.softmax(t / 0.04, dim=-1).chunk(2)
    want = sum((-tq[q] * torch.log_softmax(sv[v], -1)).sum(-1).mean() for q in range(2) for v in range(4) if v != q) / 6
    assert torch.allclose(val, want, atol=1e-5)
    assert torch.allclose(loss.center, 0.1 * t.mean(0, keepdim=True), atol=1e-6)
    sched = cosine_schedule(0.996, 1.0, 10)
    assert abs(sched[0] - 0.996) < 1e-6 and sched[-1] < 1.0 and all(sched[i] <= sched[i + 1] for i in range(9))


def test_dino_model_multi_crop_and_momentum_teacher():
    torch.manual_seed(0)
    m = DINOPretrainModel(_cfg(), img_h=32, img_w=32, patch_dim=8, out_dim=16, head_hidden=16, bottleneck=8,
                          local_crops=2, total_iters=4, freeze_last_layer_iters=1)
    for ps, pt in zip(m.student.parameters(), m.teacher.parameters()):
        assert torch.equal(ps, pt) and not pt.requires_grad
    crops = [torch.randn(3, 3, 32, 32), torch.randn(3, 3, 32, 32), torch.randn(3, 3, 16, 16), torch.randn(3, 3, 16, 16)]
    m.train()
    m.set_iteration(0)
    s, t = m(crops)
    assert s.shape == (12, 16) and t.shape == (6, 16) and not t.requires_grad
    m.dino_loss(s, t, 0).backward()
    assert m.student["head"].last_v.grad.abs().sum() == 0                     # frozen at iteration 0
    with torch.no_grad():
        for p in m.student.parameters():
            p.add_(1.0)
    before = [p.clone() for p in m.teacher.parameters()]
    m.after_optimizer_step(0)
    mom = float(m.momentum[0])
    for b, ps, pt in zip(before, m.student.parameters(), m.teacher.parameters()):
        assert torch.allclose(pt, mom * b + (1 - mom) * ps, atol=1e-6)
    m.eval()
    none, feat = m(crops[0])
    assert none is None and feat.shape == (3, 32)


def test_knn_vote():
    bank = torch.nn.functional.normalize(torch.tensor([[1.0, 0.0], [0.9, 0.1], [0.0, 1.0], [0.1, 0.9]]), dim=1).t()
    labels = torch.tensor([0, 0, 1, 1])
    q = torch.nn.functional.normalize(torch.tensor([[1.0, 0.05], [0.0, 1.0]]), dim=1)
    pred = knn_predict(q, bank, labels, classes=2, knn_k=3, knn_t=0.07)
    assert pred[:, 0].tolist() == [0, 1] and pred.shape == (2, 2)


def test_inpainting_model_masks_and_metrics():
    torch.manual_seed(0)
    m = VitInpaintingModel(_cfg(), 32, 32, 8)
    x = torch.rand(2, 3, 32, 32)
    out = m(x)
    assert out.shape == x.shape
    # the decoder of patch (i, j) writes exactly the pixels of patch (i, j)
    out.flatten(1)[0, 0].backward()
    g = m.linear_decoder.weight.grad
    assert g.abs().sum() > 0 and (g[1:].abs().sum() == 0)
    gen = torch.Generator().manual_seed(1)
    for kind in ("random", "row"):
        mask = random_patch_mask(3, 32, 32, 8, 1.0, kind, gen)
        assert mask.shape == (3, 1, 32, 32) and set(mask.unique().tolist()) <= {0.0, 1.0}
        per = mask.flatten(1).mean(1)
        assert ((per >= 0.2) & (per <= 0.3)).all()                           # a quarter of the 16 patches
        blocks = mask.view(3, 4, 8, 4, 8)
        assert (blocks.amax(dim=(2, 4)) == blocks.amin(dim=(2, 4))).all()    # whole patches only
    row = random_patch_mask(1, 32, 32, 8, 2.0, "row", gen)[0, 0]
    assert set(row.mean(dim=1).unique().tolist()) <= {0.0, 1.0} and abs(row.mean().item() - 0.5) < 1e-6
    assert psnr(x, x) > 100 and abs(psnr(x, x + 0.1).item() - 20.0) < 1e-3
    assert abs(ssim(x, x).item() - 1.0) < 1e-5 and ssim(x, torch.rand_like(x)) < 0.2
