"""The reference's extension-layer names resolve to native modules with the reference's call contracts."""
import torch
import torch.nn.functional as F

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.extensions import transformer_engine as te
from megatron_lm_b200.models.backends import LocalSpecProvider, TESpecProvider
from megatron_lm_b200.models.transformer import Norm


def _cfg(**kw):
    base = dict(num_layers=1, hidden_size=32, num_attention_heads=4, use_cpu_initialization=True,
                normalization="RMSNorm", hidden_dropout=0.0, attention_dropout=0.0)
    base.update(kw)
    return TransformerConfig(**base)


def test_norm_and_linears():
    cfg = _cfg()
    n = te.TENorm(cfg, 32, 1e-6)
    assert isinstance(n, Norm) and n.eps == 1e-6
    x = torch.randn(5, 2, 32)
    col = te.TEColumnParallelLinear(32, 48, config=cfg, init_method=cfg.init_method, bias=True, skip_bias_add=True,
                                    tp_comm_buffer_name="fc1")
    y, b = col(x)
    assert y.shape == (5, 2, 48) and b.shape == (48,) and torch.allclose(y, F.linear(x, col.weight), atol=1e-6)
    row = te.TERowParallelLinear(48, 32, config=cfg, init_method=cfg.init_method, bias=False)
    z, b2 = row(y)
    assert z.shape == (5, 2, 32) and b2 is None
    dup = te.TELinear(32, 16, parallel_mode="duplicated", config=cfg, init_method=cfg.init_method, bias=True,
                      skip_bias_add=False)
    out, b3 = dup(x)
    assert out.shape == (5, 2, 16) and b3 is None
    lnl = te.TELayerNormColumnParallelLinear(32, 48, config=cfg, init_method=cfg.init_method, bias=False)
    names = {k for k, _ in lnl.named_parameters()}
    assert "layer_norm_weight" in names and "linear.weight" in names
    ref = F.linear(F.rms_norm(x, (32,), lnl.layer_norm_weight, 1e-5), lnl.weight)
    got, _ = lnl(x)
    assert torch.allclose(got, ref, atol=1e-5)


def test_dot_product_attention_matches_sdpa():
    cfg = _cfg(num_query_groups=2)
    attn = te.TEDotProductAttention(cfg, layer_number=1, attn_mask_type="causal")
    q, k, v = torch.randn(6, 2, 4, 8), torch.randn(6, 2, 2, 8), torch.randn(6, 2, 2, 8)
    out = attn(q, k, v)
    kk, vv = k.repeat_interleave(2, dim=2), v.repeat_interleave(2, dim=2)
    ref = F.scaled_dot_product_attention(q.permute(1, 2, 0, 3), kk.permute(1, 2, 0, 3), vv.permute(1, 2, 0, 3),
                                         is_causal=True).permute(2, 0, 1, 3).reshape(6, 2, 32)
    assert torch.allclose(out, ref, atol=1e-5)
    mask = torch.zeros(2, 1, 6, 6, dtype=torch.bool)
    mask[..., 4:] = True                                                # the last two keys are padding
    full = te.TEDotProductAttention(cfg, attn_mask_type="padding")(q, k, v, attention_mask=mask)
    ref2 = F.scaled_dot_product_attention(q.permute(1, 2, 0, 3), kk.permute(1, 2, 0, 3), vv.permute(1, 2, 0, 3),
                                          attn_mask=~mask).permute(2, 0, 1, 3).reshape(6, 2, 32)
    assert torch.allclose(full, ref2, atol=1e-5)


def test_grouped_linear_and_recipe_and_helpers():
    cfg = _cfg()
    g = te.TEColumnParallelGroupedLinear(3, 32, 16, config=cfg, init_method=cfg.init_method, bias=False)
    x = torch.randn(10, 32)
    y, _ = g(x, [4, 0, 6])
    assert torch.allclose(y[:4], x[:4] @ g.weight[0].t(), atol=1e-6) and torch.allclose(y[4:], x[4:] @ g.weight[2].t(),
                                                                                       atol=1e-6)
    r = te.TEDelayedScaling(cfg, fp8_format="hybrid", amax_history_len=4, amax_compute_algo="max")
    assert r.history.numel() == 4 and r.algo == "max"
    w = torch.randn(8, 8, requires_grad=True)
    out = te.te_checkpoint(lambda t: (t * w).sin(), False, None, None, torch.randn(8, 8, requires_grad=True))
    out.sum().backward()
    assert w.grad is not None
    ctx, sync = te.get_cpu_offload_context(False, 2, 2, True, False)
    with ctx:
        assert sync(out) is out
    assert te.HAVE_TE is False


def test_spec_providers_answer_with_native_classes():
    loc, tep = LocalSpecProvider(), TESpecProvider()
    assert not loc.fuse_layernorm_and_linear() and loc.column_parallel_layer_norm_linear() is None
    assert tep.fuse_layernorm_and_linear() and tep.column_parallel_layer_norm_linear() is te.TELayerNormColumnParallelLinear
    assert tep.column_parallel_linear() is te.TEColumnParallelLinear and tep.row_parallel_linear() is te.TERowParallelLinear
    assert loc.core_attention() is te.TEDotProductAttention and loc.layer_norm() is Norm
    cls, sub = loc.grouped_mlp_modules(True, False)
    assert cls.__name__ == "GroupedMLP" and sub is None
    cls, sub = tep.grouped_mlp_modules(False, False)
    assert cls.__name__ == "SequentialMLP" and sub.linear_fc1 is te.TEColumnParallelLinear


def test_remaining_adapter_names_and_small_helpers():
    """TEFusedMLP, the RNG tracker name, SplitAlongDim, the rotary entry, the general GEMM in the library's
    convention; multi-tensor fallbacks, routing-map padding, frozen-weight linear, YAML helpers, the
    context-parallel slice of a position table."""
    import torch
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.extensions import transformer_engine as te
    from megatron_lm_b200.models.moe import pad_routing_map
    from megatron_lm_b200.models.position_embeddings import get_pos_emb_on_this_cp_rank
    from megatron_lm_b200.parallel.layers import LinearWithFrozenWeight
    from megatron_lm_b200.utils.common import (local_multi_tensor_applier, local_multi_tensor_l2_norm,
                                               local_multi_tensor_scale)
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            use_cpu_initialization=True)
    mlp = te.TEFusedMLP(cfg)
    y, _ = mlp(torch.randn(5, 2, 32))
    assert y.shape == (5, 2, 32)
    assert not te.TECudaRNGStatesTracker().is_initialized()
    a, b = te.SplitAlongDim(torch.arange(12.0).view(2, 6), 1, (2, 4))
    assert a.shape == (2, 2) and b.shape == (2, 4)
    A, B = torch.randn(7, 16), torch.randn(5, 16)                       # TN: B @ A^T
    out = te.te_general_gemm(A, B, torch.float32, layout="TN")[0]
    assert torch.allclose(out, B @ A.t(), atol=1e-5)
    t = torch.randn(6, 2, 4, 8)
    f = torch.randn(6, 1, 1, 4)
    freqs = torch.cat((f, f), dim=-1)
    rot = te.fused_apply_rotary_pos_emb(t, freqs)
    half = t.shape[-1] // 2
    ang = freqs.reshape(6, -1)
    cos, sin = torch.cos(ang)[:, None, None, :], torch.sin(ang)[:, None, None, :]
    rotated = torch.cat((-t[..., half:], t[..., :half]), dim=-1)
    assert torch.allclose(rot, t * cos + rotated * sin, atol=1e-5)
    # multi-tensor fallbacks
    ts = [torch.randn(5), torch.randn(3, 4)]
    total, per = local_multi_tensor_applier(local_multi_tensor_l2_norm, None, [ts], True)
    assert torch.allclose(total, torch.cat([x.flatten() for x in ts]).norm().reshape(1)) and per.shape == (2,)
    dst = [torch.zeros(5), torch.zeros(3, 4)]
    local_multi_tensor_applier(local_multi_tensor_scale, None, [ts, dst], 0.5)
    assert torch.allclose(dst[1], ts[1] * 0.5)
    # routing-map padding: every expert's count becomes a multiple of 4, earlier choices stay
    rm = torch.zeros(10, 3, dtype=torch.bool)
    rm[[0, 3, 4], 0] = True
    rm[:, 1] = True
    padded = pad_routing_map(rm, 4)
    assert padded.sum(0).tolist() == [4, 10, 0] and (padded | rm).equal(padded) and padded[1, 0]
    # frozen weight
    w = torch.randn(6, 4, requires_grad=True)
    x = torch.randn(3, 4, requires_grad=True)
    LinearWithFrozenWeight.apply(x, w).sum().backward()
    assert w.grad is None and x.grad is not None
    # context-parallel rows of a table
    tab = torch.arange(16.0).view(16, 1)
    assert get_pos_emb_on_this_cp_rank(tab, 0, 2, 0).flatten().tolist() == [0, 1, 2, 3, 12, 13, 14, 15]
    assert get_pos_emb_on_this_cp_rank(tab, 0, 2, 1).flatten().tolist() == [4, 5, 6, 7, 8, 9, 10, 11]
    assert get_pos_emb_on_this_cp_rank(tab, 0, 1, 0) is tab
