"""Sampling kernel against the PyTorch statement of the same rule (same uniforms -> same tokens)."""
import pytest
import torch

from megatron_lm_b200.ops import sampling as S

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V", [1000, 32000, 50257])
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 1, 0.0), (0.7, 40, 0.0), (1.3, 0, 0.9), (1.0, 0, 0.0)])
def test_sample_matches_reference(dtype, V, temperature, top_k, top_p):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.manual_seed(V + top_k)
    rows = 64
    lg = (3.0 * torch.randn(rows, V, device="cuda")).to(dtype)
    u = torch.rand(rows, device="cuda")
    got = S.sample(lg, u, temperature, top_k, top_p)
    want = S.sample_reference(lg, u, temperature, top_k, top_p)
    assert got.dtype == torch.int64 and got.shape == (rows,)
    kept = S._kept_probs(lg, temperature, top_k, top_p) > 0 if top_k != 1 else None
    if kept is not None:
        assert bool(kept.gather(1, got.view(-1, 1)).all()), "a filtered-out token was drawn"
    # equal except where the running sums round differently right at a boundary
    assert (got == want).float().mean() >= 0.95, (got, want)


def test_sample_distribution():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.manual_seed(0)
    lg = torch.randn(1, 12, device="cuda").expand(40000, 12).contiguous()
    tok = S.sample(lg, torch.rand(40000, device="cuda"), 0.9, 0, 0.0)
    emp = torch.bincount(tok, minlength=12).float() / 40000
    assert (emp - (lg[0] / 0.9).softmax(-1)).abs().max() < 0.01


def test_engine_sampler_uses_kernel_and_generator():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from megatron_lm_b200.inference.engine import SamplingParams, sample_from_logits
    lg = torch.randn(8, 5000, device="cuda")
    g1 = torch.Generator(device="cuda").manual_seed(5)
    g2 = torch.Generator(device="cuda").manual_seed(5)
    a = sample_from_logits(lg, SamplingParams(temperature=0.8, top_k=50), generator=g1)
    b = sample_from_logits(lg, SamplingParams(temperature=0.8, top_k=50), generator=g2)
    assert torch.equal(a, b)
    top = torch.topk(lg, 50, dim=-1).indices
    assert bool((top == a.view(-1, 1)).any(-1).all())
    assert torch.equal(sample_from_logits(lg, SamplingParams(top_k=1)), lg.argmax(-1))
