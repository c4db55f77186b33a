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


def _mamba_cp_rank(rank, world, pattern, out_path):
    """A (hybrid) Mamba model on a context-parallel group reproduces the logits and - summed over the group - the
    gradients of the single-process model on the full sequence."""
    import torch.distributed as dist
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.mamba import MambaModel
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.context_parallel import zigzag_indices
    cp = world
    state.initialize_model_parallel(context_parallel_size=cp)
    S, b = 32, 2

    def build(cp_size):
        torch.manual_seed(11)
        cfg = TransformerConfig(num_layers=len(pattern), hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                                hidden_dropout=0.0, attention_dropout=0.0, normalization="RMSNorm", add_bias_linear=False,
                                context_parallel_size=cp_size, use_cpu_initialization=True)
        return MambaModel(cfg, 48, S, hybrid_override_pattern=pattern, d_state=8, headdim=16, ngroups=2, chunk_size=8,
                          position_embedding_type="rope", parallel_output=False)
    ids = torch.randint(0, 48, (b, S), generator=torch.Generator().manual_seed(5))
    w = torch.randn(b, S, 48, generator=torch.Generator().manual_seed(6))
    model = build(cp)
    idx = zigzag_indices(S, cp, rank)
    out = model(ids[:, idx])
    (out * w[:, idx]).sum().backward()
    grads = {}
    for n, p in model.named_parameters():
        g = p.grad.clone() if p.grad is not None else torch.zeros_like(p)
        dist.all_reduce(g, group=state.get_context_parallel_group())
        grads[n] = g
    if rank == 0:
        # the full-sequence model in the same process: the group is left aside by giving the mixers cp = 1
        state.destroy_model_parallel()
        state.initialize_model_parallel(context_parallel_size=1, tensor_model_parallel_size=1) if False else None
    torch.save({"out": out.detach(), "idx": idx, "grads": grads}, f"{out_path}.{rank}")


def _mamba_full(pattern):
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.mamba import MambaModel
    S, b = 32, 2
    torch.manual_seed(11)
    cfg = TransformerConfig(num_layers=len(pattern), hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, normalization="RMSNorm", add_bias_linear=False,
                            use_cpu_initialization=True)
    model = MambaModel(cfg, 48, S, hybrid_override_pattern=pattern, d_state=8, headdim=16, ngroups=2, chunk_size=8,
                       position_embedding_type="rope", parallel_output=False)
    ids = torch.randint(0, 48, (b, S), generator=torch.Generator().manual_seed(5))
    w = torch.randn(b, S, 48, generator=torch.Generator().manual_seed(6))
    out = model(ids)
    (out * w).sum().backward()
    return out.detach(), {n: p.grad.clone() for n, p in model.named_parameters()}


@pytest.mark.parametrize("pattern", ["MM", "M*-M"])
def test_mamba_context_parallel_matches_full_sequence(tmp_path, pattern):
    path = str(tmp_path / "m")
    run_distributed(_mamba_cp_rank, 2, pattern, path)
    ref_out, ref_grads = _mamba_full(pattern)
    for r in range(2):
        got = torch.load(f"{path}.{r}")
        assert torch.allclose(got["out"], ref_out[:, got["idx"]], atol=2e-5), (got["out"] - ref_out[:, got["idx"]]).abs().max()
        for n, g in got["grads"].items():
            assert torch.allclose(g, ref_grads[n], atol=2e-4, rtol=1e-3), (n, (g - ref_grads[n]).abs().max())
