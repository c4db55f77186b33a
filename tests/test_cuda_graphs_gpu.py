"""Graph-captured transformer layer equals the eager layer (outputs, input gradient, weight gradients)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_graphed_layer_matches_eager():
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.transformer import TransformerLayer
    from megatron_lm_b200.utils.cuda_graphs import FullIterationGraph, GraphedModule
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=1, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512,
                            hidden_dropout=0.0, attention_dropout=0.0, params_dtype=torch.bfloat16, bf16=True,
                            normalization="RMSNorm", gated_linear_unit=True, add_bias_linear=False,
                            use_cpu_initialization=False)
    layer = TransformerLayer(cfg, 1).cuda()
    for p in layer.parameters():
        p.main_grad = torch.zeros_like(p, dtype=torch.float32)
    x = torch.randn(128, 2, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(128, 2, 256, device="cuda", dtype=torch.bfloat16)
    y = layer(x)
    y.backward(g)
    ref_y, ref_dx = y.detach().clone(), x.grad.clone()
    ref_w = [p.main_grad.clone() for p in layer.parameters()]
    for p in layer.parameters():
        p.main_grad.zero_()
    # the eager graph (and the gradient-accumulation nodes it created on this stream) must be gone before capture
    del y
    x.grad = None
    gl = GraphedModule(layer)
    for it in range(2):                       # second call replays
        x2 = x.detach().clone().requires_grad_()
        y2 = gl(x2)
        y2.backward(g)
        assert torch.allclose(y2.float(), ref_y.float(), atol=2e-2, rtol=2e-2)
        assert torch.allclose(x2.grad.float(), ref_dx.float(), atol=2e-2, rtol=2e-2)
        for p, r in zip(layer.parameters(), ref_w):
            assert torch.allclose(p.main_grad, r * (it + 1), atol=5e-2, rtol=5e-2)
    f = FullIterationGraph(lambda a, b: a * 2 + b)
    a, b = torch.ones(4, device="cuda"), torch.ones(4, device="cuda")
    assert f(a, b).tolist() == [3.0] * 4
    assert f(a * 2, b).tolist() == [5.0] * 4
