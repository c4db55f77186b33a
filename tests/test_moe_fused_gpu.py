"""MoE layer with the peer-memory dispatch/combine kernels equals the NCCL all-to-all dispatcher
(outputs, input gradient, router and expert weight gradients) on 2 and 4 GPUs."""
import pytest
import torch

from tests.gpu_dist_utils import run_on_gpus

pytestmark = pytest.mark.gpu


def _worker(rank, world):
    import torch.distributed as dist
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.moe import MoELayer
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.random import model_parallel_cuda_manual_seed
    state.initialize_model_parallel(expert_model_parallel_size=world, create_gloo_process_groups=False)
    outs = {}
    for kind in ("alltoall", "flex"):
        model_parallel_cuda_manual_seed(11)          # same expert initialisation for both layers
        torch.manual_seed(5)
        cfg = TransformerConfig(num_layers=1, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512,
                                num_moe_experts=2 * world, moe_router_topk=2, moe_ffn_hidden_size=256,
                                moe_token_dispatcher_type=kind, moe_grouped_gemm=True, moe_aux_loss_coeff=0.0,
                                expert_model_parallel_size=world, params_dtype=torch.bfloat16, bf16=True,
                                gated_linear_unit=True, add_bias_linear=False, use_cpu_initialization=False,
                                hidden_dropout=0.0, attention_dropout=0.0)
        layer = MoELayer(cfg, 1).cuda()
        for p in layer.parameters():
            p.main_grad = torch.zeros_like(p, dtype=torch.float32)
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        x = torch.randn(192, 2, 256, device="cuda", generator=g).bfloat16().requires_grad_()
        gy = torch.randn(192, 2, 256, device="cuda", generator=g).bfloat16()
        y, _ = layer(x)
        y.backward(gy)
        grads = {n: (p.main_grad.clone() if p.grad is None else p.grad.float() + p.main_grad)
                 for n, p in layer.named_parameters()}
        outs[kind] = (y.detach().float(), x.grad.float(), grads)
    ya, xa, ga = outs["alltoall"]
    yf, xf, gf = outs["flex"]
    assert torch.allclose(ya, yf, atol=2e-2, rtol=2e-2), (ya - yf).abs().max()
    assert torch.allclose(xa, xf, atol=2e-2, rtol=2e-2), (xa - xf).abs().max()
    for n in ga:
        assert torch.allclose(ga[n], gf[n], atol=3e-2, rtol=3e-2), (n, (ga[n] - gf[n]).abs().max())


@pytest.mark.parametrize("world", [2, 4])
def test_fused_dispatcher_matches_alltoall(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_on_gpus(_worker, world)
