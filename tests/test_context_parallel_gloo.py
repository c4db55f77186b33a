"""Ring / all-gather / Ulysses context-parallel attention on Gloo ranks against full-sequence attention."""
import math

import pytest
import torch

from tests.dist_utils import run_distributed


def _run(rank, world, kind, ng, qpg):
    import torch.distributed as dist
    from megatron_lm_b200.ops.attention import _ref_attention
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.context_parallel import context_parallel_attention, zigzag_indices
    state.initialize_model_parallel(context_parallel_size=world,
                                    hierarchical_context_parallel_sizes=[2, world // 2] if kind == "a2a+p2p" else None)
    torch.manual_seed(3)
    S, b, d = 16 * world, 2, 8
    q = torch.randn(S, b, ng, qpg, d, dtype=torch.float64)
    k = torch.randn(S, b, ng, d, dtype=torch.float64)
    v = torch.randn(S, b, ng, d, dtype=torch.float64)
    do = torch.randn(S, b, ng * qpg, d, dtype=torch.float64)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    ref = _ref_attention(qr, kr, vr, True, 1 / math.sqrt(d)).double()
    ref.backward(do)
    idx = zigzag_indices(S, world, rank)
    ql, kl, vl = (t[idx].clone().requires_grad_() for t in (q, k, v))
    out = context_parallel_attention(ql, kl, vl, kind, state.get_context_parallel_group())
    assert torch.allclose(out.double(), ref[idx].detach(), atol=1e-5), (kind, (out - ref[idx]).abs().max())
    out.backward(do[idx].to(out.dtype))
    assert torch.allclose(ql.grad, qr.grad[idx], atol=1e-5)
    assert torch.allclose(kl.grad, kr.grad[idx], atol=1e-5), (kl.grad - kr.grad[idx]).abs().max()
    assert torch.allclose(vl.grad, vr.grad[idx], atol=1e-5)


@pytest.mark.parametrize("kind", ["p2p", "all_gather", "a2a"])
@pytest.mark.parametrize("world", [2, 4])
def test_cp_attention_matches_full(kind, world):
    run_distributed(_run, world, kind, 4, 2)


def test_hierarchical_a2a_p2p_matches_full():
    """cp = 4 as 2 (all-to-all inside a pair of ranks) x 2 (ring between the pairs)."""
    run_distributed(_run, 4, "a2a+p2p", 4, 2)
