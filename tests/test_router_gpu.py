"""Fused MoE router kernel against the plain PyTorch fp32 body of the same op."""
import pytest
import torch

from megatron_lm_b200.ops import router as R

pytestmark = pytest.mark.gpu


def _explicit(lg, topk, mode, scale, bias, w, aux_coeff, z_coeff, ls):
    T, E = lg.shape
    lg = lg.detach().clone().requires_grad_(True)
    pr, rm, tpe, ss, zs = R._reference(lg, topk, mode, scale, bias)
    aux = (ss * tpe.float()).sum() * (aux_coeff * E / (T * T * topk))
    z = zs * (z_coeff / T)
    ((pr * w).sum() + ls * (aux + z)).backward()
    return pr.detach(), rm, tpe, aux.detach(), z.detach(), lg.grad


@pytest.mark.parametrize("mode", ["softmax_post", "softmax_pre", "sigmoid"])
@pytest.mark.parametrize("E,topk", [(8, 2), (3, 1), (16, 2), (24, 3), (64, 6), (128, 4), (160, 1), (256, 8), (300, 2),
                                    (600, 4)])
def test_router_kernel_matches_reference(mode, E, topk):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.manual_seed(E * 7 + topk)
    T = 1003 if E != 3 else 5          # not a multiple of the tokens a warp takes at a time; fewer tokens than lanes
    lg = torch.randn(T, E, device="cuda", requires_grad=True)
    bias = 0.1 * torch.randn(E, device="cuda") if mode == "sigmoid" else None
    w = torch.randn(T, E, device="cuda")
    ls = torch.tensor(3.0, device="cuda")
    p, m, tpe, aux, z = R.fused_topk_router(lg, topk, mode, 1.25, bias, aux_coeff=0.01, z_coeff=0.001,
                                            loss_scale=lambda: ls)
    (p * w).sum().backward()
    pr, rm, t2, a2, z2, g2 = _explicit(lg, topk, mode, 1.25, bias, w, 0.01, 0.001, 3.0)
    assert m.dtype == torch.bool and torch.equal(m, rm)
    assert torch.equal(tpe, t2)
    assert torch.allclose(p, pr, rtol=1e-4, atol=1e-6)
    assert torch.allclose(aux, a2, rtol=1e-4) and torch.allclose(z, z2, rtol=1e-4)
    assert torch.allclose(lg.grad, g2, rtol=2e-4, atol=1e-6), (lg.grad - g2).abs().max()


def test_router_module_fused_equals_unfused(monkeypatch):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.moe import TopKRouter
    cfg = TransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, num_moe_experts=8,
                            moe_router_topk=2, moe_aux_loss_coeff=0.01, moe_z_loss_coeff=0.001,
                            moe_router_load_balancing_type="aux_loss", use_cpu_initialization=False)
    torch.manual_seed(1)
    r = TopKRouter(cfg, 1).cuda().train()
    x = torch.randn(16, 4, 64, device="cuda")
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("MLB_FUSED_ROUTER", flag)
        r.zero_grad()
        p, m = r(x)
        (p * p).sum().backward()
        outs.append((p.detach().clone(), m.clone(), r.weight.grad.clone()))
    assert torch.equal(outs[0][1], outs[1][1])
    assert torch.allclose(outs[0][0], outs[1][0], rtol=1e-4, atol=1e-6)
    assert torch.allclose(outs[0][2], outs[1][2], rtol=1e-3, atol=1e-6)
