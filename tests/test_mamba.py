"""State-space ops against the step-by-step recurrence; Mamba model trains and decodes incrementally."""
import pytest
import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.mamba import MambaInferenceCache, MambaModel, allocate_layers
from megatron_lm_b200.ops.mamba import _conv_ref, causal_conv1d, ssd_chunked, ssd_reference, ssd_scan


def _rand(b=2, l=70, H=4, P=8, G=2, N=16, device="cpu", dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(b, l, H, P, generator=g).to(device, dtype)
    dt = torch.rand(b, l, H, generator=g).to(device) * 0.5 + 0.01
    A = -(torch.rand(H, generator=g).to(device) * 2 + 0.5)
    Bm = torch.randn(b, l, G, N, generator=g).to(device, dtype) * 0.5
    Cm = torch.randn(b, l, G, N, generator=g).to(device, dtype) * 0.5
    D = torch.randn(H, generator=g).to(device)
    return x, dt, A, Bm, Cm, D


def test_chunked_ssd_matches_recurrence():
    x, dt, A, Bm, Cm, D = _rand()
    y_ref, h_ref = ssd_reference(x, dt, A, Bm, Cm, D)
    y, h = ssd_chunked(x, dt, A, Bm, Cm, D, chunk=16)
    assert torch.allclose(y, y_ref, atol=1e-4, rtol=1e-4) and torch.allclose(h, h_ref, atol=1e-4, rtol=1e-4)
    # continuing from a state equals one long scan
    y1, h1 = ssd_chunked(x[:, :40], dt[:, :40], A, Bm[:, :40], Cm[:, :40], D, chunk=16)
    y2, h2 = ssd_chunked(x[:, 40:], dt[:, 40:], A, Bm[:, 40:], Cm[:, 40:], D, chunk=16, initial_state=h1)
    assert torch.allclose(torch.cat((y1, y2), 1), y_ref, atol=1e-4, rtol=1e-4)


def test_hybrid_allocation():
    assert allocate_layers(4, override_pattern="M*-M") == ["M", "*", "-", "M"]
    lay = allocate_layers(8, 0.25, 0.25)
    assert lay.count("*") == 2 and lay.count("-") == 2 and lay.count("M") == 4
    with pytest.raises(ValueError):
        allocate_layers(3, override_pattern="MX*")


def _model(device="cpu", dtype=torch.float32):
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=3, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, normalization="RMSNorm", add_bias_linear=False,
                            params_dtype=dtype, bf16=dtype == torch.bfloat16)
    return MambaModel(cfg, 64, 64, hybrid_override_pattern="M-M", d_state=16, headdim=16, ngroups=2,
                      chunk_size=8).to(device)


def test_mamba_model_trains_and_decodes():
    m = _model()
    ids = torch.randint(0, 64, (2, 20))
    m(ids, labels=ids).mean().backward()
    for n, p in m.named_parameters():
        g = p.grad if p.grad is not None else getattr(p, "main_grad", None)
        assert g is not None and torch.isfinite(g).all(), n
    m.eval()
    with torch.no_grad():
        full = m(ids)
        cache = MambaInferenceCache()
        outs = [m(ids[:, :12], inference_context=cache)]
        for t in range(12, 20):
            outs.append(m(ids[:, t:t + 1], inference_context=cache))
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
def test_mamba_kernels_gpu():
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        x, dt, A, Bm, Cm, D = _rand(b=2, l=100, H=4, P=64, G=2, N=128, device="cuda", dtype=dtype)
        y_ref, h_ref = ssd_reference(x, dt, A, Bm, Cm, D)
        st = torch.zeros(2, 4, 64, 128, device="cuda")
        with torch.no_grad():
            y = ssd_scan(x, dt, A, Bm, Cm, D, None, st, False)
        assert torch.allclose(y.float(), y_ref, atol=tol * 10, rtol=tol), (y.float() - y_ref).abs().max()
        assert torch.allclose(st, h_ref, atol=tol * 10, rtol=tol)
        # conv forward / backward against the fp32 conv
        xc = torch.randn(2, 150, 96, device="cuda", dtype=dtype, requires_grad=True)
        w = torch.randn(96, 4, device="cuda", dtype=dtype, requires_grad=True)
        bias = torch.randn(96, device="cuda", dtype=dtype, requires_grad=True)
        y = causal_conv1d(xc, w, bias, True)
        gy = torch.randn_like(y)
        y.backward(gy)
        x2, w2, b2 = (t.detach().float().requires_grad_() for t in (xc, w, bias))
        y2 = _conv_ref(x2, w2, b2, True)
        y2.backward(gy.float())
        assert torch.allclose(y.float(), y2, atol=tol * 5, rtol=tol)
        assert torch.allclose(xc.grad.float(), x2.grad, atol=tol * 10, rtol=tol * 2)
        assert torch.allclose(w.grad.float(), w2.grad, atol=tol * 60, rtol=tol * 2)
        assert torch.allclose(bias.grad.float(), b2.grad, atol=tol * 60, rtol=tol * 2)


@pytest.mark.gpu
@pytest.mark.parametrize("C,G", [(256, 1), (1024, 8), (4096, 2), (2560, 5), (8192, 8), (16384, 4)])
def test_gated_rmsnorm_gpu(C, G):
    from megatron_lm_b200.ops.mamba import _gated_rmsnorm_ref, gated_rmsnorm
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        torch.manual_seed(C + G)
        big = torch.randn(3, 70, 2 * C + 64, device="cuda", dtype=dtype)
        z = big[..., :C].detach().requires_grad_()                  # strided slice, as in the mixer
        y = torch.randn(3, 70, C, device="cuda", dtype=dtype, requires_grad=True)
        w = (1 + 0.1 * torch.randn(C, device="cuda")).requires_grad_()
        out = gated_rmsnorm(y, z, w, G, 1e-5)
        g = torch.randn_like(out)
        out.backward(g)
        y2, z2, w2 = (t.detach().float().requires_grad_() for t in (y, z, w))
        ref = _gated_rmsnorm_ref(y2, z2, w2, G, 1e-5)
        ref.backward(g.float())
        assert torch.allclose(out.float(), ref, atol=tol * 4, rtol=tol)
        assert torch.allclose(y.grad.float(), y2.grad, atol=tol * 8, rtol=tol * 2)
        assert torch.allclose(z.grad.float(), z2.grad, atol=tol * 8, rtol=tol * 2)
        assert torch.allclose(w.grad.float(), w2.grad, atol=tol * 200, rtol=tol * 4)


@pytest.mark.parametrize("pattern,pos", [("M-M", "none"), ("M*-M", "rope"), ("M*M-", "learned_absolute")])
def test_mamba_and_hybrid_models_generate_through_the_static_engine(pattern, pos):
    """Prompts of different lengths in one batch: state-space states advance token by token with the forced prompt
    tokens, attention layers of hybrids use the engine's key / value cache with the right positions."""
    from megatron_lm_b200.inference import DynamicInferenceEngine, SamplingParams, StaticInferenceEngine
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=len(pattern), hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, normalization="RMSNorm", add_bias_linear=False)
    m = MambaModel(cfg, 64, 64, hybrid_override_pattern=pattern, d_state=16, headdim=16, ngroups=2, chunk_size=8,
                   position_embedding_type=pos).eval()
    prompts = [[5, 9, 2, 33, 7, 1, 4], [11, 4, 6]]
    out = StaticInferenceEngine(m, max_batch_size=2, max_sequence_length=32).generate(
        prompts, SamplingParams(top_k=1, num_tokens_to_generate=6))
    for req, p in zip(out, prompts):
        toks = list(p)
        with torch.no_grad():
            for _ in range(len(req.generated_tokens)):
                toks.append(int(m(torch.tensor([toks]))[0, -1].float().argmax()))
        assert req.generated_tokens == toks[len(p):], (pattern, req.generated_tokens, toks[len(p):])
    with pytest.raises(NotImplementedError):
        DynamicInferenceEngine(m, max_requests=2, max_sequence_length=32, chunk_size=4).generate(
            prompts, SamplingParams(top_k=1, num_tokens_to_generate=2))
