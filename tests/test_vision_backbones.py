"""MiT and Swin backbones and the models on top of them (reference: megatron/legacy/model/vision/mit_backbone.py,
esvit_swin_backbone.py, classification.py:58, inpainting.py:84, dino.py:179-215)."""
import pytest
import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models import vision_backbones as vb
from megatron_lm_b200.models.vision_backbones import (
    MitClassificationModel, MitInpaintingModel, MixVisionTransformer, SwinTransformer, _SwinBlock, _unwindows, _windows)


def _cfg(**kw):
    base = dict(num_layers=2, hidden_size=64, num_attention_heads=4, use_cpu_initialization=True,
                params_dtype=torch.float32, hidden_dropout=0.0, attention_dropout=0.0)
    base.update(kw)
    return TransformerConfig(**base)


def test_mit_feature_maps_and_average():
    torch.manual_seed(0)
    m = MixVisionTransformer.preset("b0", drop_path_rate=0.0)
    x = torch.randn(2, 3, 64, 64)
    maps = m(x)
    assert [tuple(t.shape) for t in maps] == [(2, 32, 16, 16), (2, 64, 8, 8), (2, 160, 4, 4), (2, 256, 2, 2)]
    avg = MixVisionTransformer.preset("b0", drop_path_rate=0.0, output_avg=True)
    avg.load_state_dict(m.state_dict())
    torch.testing.assert_close(avg(x), maps[3].flatten(2).mean(-1))
    # depths of the larger presets
    assert [len(s.blocks) for s in MixVisionTransformer.preset("b3").stages] == [3, 4, 18, 3]


def test_mit_reduced_attention_matches_explicit_softmax():
    torch.manual_seed(1)
    att = vb._ReducedAttention(64, 2, 2, True, {})
    x = torch.randn(2, 16, 64)
    out = att(x, (4, 4))
    # the same by hand: keys / values from the 2 x 2 map
    q = att.q(x).view(2, 16, 2, 32).transpose(1, 2)
    m = att.reduce_norm(att.reduce(x.transpose(1, 2).reshape(2, 64, 4, 4)).flatten(2).transpose(1, 2))
    assert m.shape == (2, 4, 64)
    k, v = att.kv(m).view(2, 4, 2, 2, 32).permute(2, 0, 3, 1, 4)
    p = torch.softmax(q @ k.transpose(-1, -2) / 32 ** 0.5, dim=-1)
    torch.testing.assert_close(out, att.proj((p @ v).transpose(1, 2).reshape(2, 16, 64)))


def test_window_partition_round_trip_and_shift_mask():
    x = torch.arange(2 * 8 * 12 * 3, dtype=torch.float32).view(2, 8, 12, 3)
    w = _windows(x, 4)
    assert w.shape == (2 * 2 * 3, 16, 3)
    torch.testing.assert_close(_unwindows(w, 4, 2, 8, 12), x)
    torch.testing.assert_close(w[1, :, 0].view(4, 4), x[0, :4, 4:8, 0])
    blk = _SwinBlock(16, 2, 4, True, 2.0, True, 0.0, {})
    mask = blk._shift_mask(8, 8, 4, 2, torch.device("cpu"))
    assert mask.shape == (4, 16, 16)
    assert (mask[0] == 0).all()                              # the top-left window holds one region only
    assert (mask[3] != 0).any() and (mask[3].diagonal() == 0).all()
    # the last window is four regions of 2 x 2 tokens: each token sees exactly its own region
    assert ((mask[3] == 0).sum(-1) == 4).all()


def test_swin_block_is_shift_equivariant_without_borders():
    """A block with shifted windows on a cyclically shifted image equals the shifted output of the unshifted-window
    block, as long as no masking is involved (mask zeroed)."""
    torch.manual_seed(2)
    plain = _SwinBlock(16, 2, 4, False, 2.0, True, 0.0, {})
    shifted = _SwinBlock(16, 2, 4, True, 2.0, True, 0.0, {})
    shifted.load_state_dict(plain.state_dict())
    x = torch.randn(1, 8, 8, 16)
    shifted._masks[(8, 8, 4, 2, "cpu")] = torch.zeros(4, 16, 16)
    out_s = shifted(x.reshape(1, 64, 16), (8, 8)).view(1, 8, 8, 16)
    rolled = torch.roll(x, shifts=(-2, -2), dims=(1, 2))
    out_p = plain(rolled.reshape(1, 64, 16), (8, 8)).view(1, 8, 8, 16)
    torch.testing.assert_close(out_s, torch.roll(out_p, shifts=(2, 2), dims=(1, 2)), atol=1e-5, rtol=1e-5)


def test_swin_shapes_small_maps_and_padding():
    torch.manual_seed(3)
    m = SwinTransformer(width=16, depths=(2, 2, 2, 2), heads=(2, 2, 4, 4), window=4, drop_path_rate=0.0)
    assert m.num_features == 128
    assert m(torch.randn(2, 3, 96, 96)).shape == (2, 128)          # 24 -> 12 -> 6 -> 3 (smaller than the window)
    assert m(torch.randn(2, 3, 72, 40)).shape == (2, 128)          # 18 x 10: padded to multiples of the window
    maps = SwinTransformer(width=16, depths=(1, 1, 1, 1), heads=(2, 2, 4, 4), window=4, output_avg=False)
    assert maps(torch.randn(1, 3, 64, 64)).shape == (1, 128, 2, 2)
    full = SwinTransformer.preset("tiny")
    assert full.num_features == 768 and [len(b) for b in full.blocks] == [2, 2, 6, 2]
    # a window that covers the whole map sees every token: the output does not depend on the padding of others
    loss = m(torch.randn(2, 3, 64, 64)).sum()
    loss.backward()
    assert all(p.grad is not None for p in m.parameters())


def test_mit_classifier_learns_and_inpainting_shape():
    torch.manual_seed(4)
    cfg = _cfg()
    clf = MitClassificationModel(cfg, 4, preset="b0")
    for mod in clf.modules():
        if isinstance(mod, vb.DropPath):
            mod.p = 0.0
    x = torch.randn(8, 3, 32, 32)
    y = torch.arange(8) % 4
    x = x + y.view(8, 1, 1, 1).float()                                # the class is the brightness
    opt = torch.optim.AdamW(clf.parameters(), lr=2e-3)
    first = None
    for _ in range(30):
        loss = torch.nn.functional.cross_entropy(clf(x), y)
        first = first if first is not None else float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < 0.5 * first
    inp = MitInpaintingModel(cfg, 32, 32, 4, preset="b0", embed=32)
    out = inp(torch.randn(2, 3, 32, 32))
    assert out.shape == (2, 3, 32, 32)
    out.sum().backward()
    assert inp.predict.weight.grad is not None and inp.backbone.stages[0].embed.weight.grad is not None
    with pytest.raises(ValueError, match="4 x 4"):
        MitInpaintingModel(cfg, 32, 32, 8, preset="b0")


def test_dino_towers_on_hierarchical_backbones(monkeypatch):
    from megatron_lm_b200.models.vision import DINOPretrainModel
    monkeypatch.setitem(vb.SWIN_PRESETS, "tiny", (16, (1, 1, 1, 1), (2, 2, 4, 4), 0.1))
    monkeypatch.setitem(vb.MIT_PRESETS, "b5", ((16, 32, 32, 64), (1, 2, 2, 4), (1, 1, 1, 1)))
    for kind, width in (("swin", 128), ("mit", 64)):
        torch.manual_seed(5)
        m = DINOPretrainModel(_cfg(), img_h=64, img_w=64, patch_dim=4, out_dim=32, head_hidden=32, bottleneck=16,
                              local_crops=2, total_iters=4, backbone_type=kind)
        crops = [torch.randn(2, 3, 64, 64), torch.randn(2, 3, 64, 64), torch.randn(2, 3, 32, 32), torch.randn(2, 3, 32, 32)]
        s_out, t_out = m(crops)
        assert s_out.shape == (8, 32) and t_out.shape == (4, 32)
        loss = m.dino_loss(s_out, t_out, 0)
        loss.backward()
        m.after_optimizer_step(0)
        m.eval()
        assert m(crops[0])[1].shape == (2, width)
        # the teacher has no stochastic depth, the student does
        t_rates = [mod.p for mod in m.teacher.modules() if isinstance(mod, vb.DropPath)]
        s_rates = [mod.p for mod in m.student.modules() if isinstance(mod, vb.DropPath)]
        assert max(t_rates) == 0.0 and max(s_rates) > 0.0


@pytest.mark.gpu
def test_mit_and_swin_on_gpu_match_cpu_reference():
    """The same weights on the GPU and on the host: fp32 agrees closely (forward and input gradient), bf16 stays
    within the precision of the format."""
    torch.manual_seed(6)
    x = torch.randn(2, 3, 64, 64)
    for build in (lambda **kw: MixVisionTransformer(widths=(64, 128, 128, 128), heads=(1, 2, 2, 2), depths=(1, 1, 1, 1),
                                                    drop_path_rate=0.0, output_avg=True, **kw),
                  lambda **kw: SwinTransformer(width=32, depths=(2, 1, 1, 1), heads=(2, 2, 4, 4), window=4,
                                               drop_path_rate=0.0, **kw)):
        ref = build()
        xr = x.clone().requires_grad_(True)
        out_r = ref(xr)
        out_r.sum().backward()
        dev = build(device="cuda", dtype=torch.float32)
        dev.load_state_dict(ref.state_dict())
        xd = x.cuda().requires_grad_(True)
        out_d = dev(xd)
        out_d.sum().backward()
        torch.testing.assert_close(out_d.cpu(), out_r, atol=2e-2, rtol=2e-2)       # convolutions may run in TF32
        assert torch.nn.functional.cosine_similarity(xr.grad.flatten(), xd.grad.cpu().flatten(), dim=0) > 0.99
        half = build(device="cuda", dtype=torch.bfloat16)
        half.load_state_dict(ref.state_dict())
        out_h = half(x.cuda()).float().cpu()
        assert torch.isfinite(out_h).all()
        assert (out_h - out_r).norm() / out_r.norm() < 0.2
