"""Each CUDA op against the plain-PyTorch fp32 body of the same op."""
import pytest
import torch

from megatron_lm_b200.ops import core, optim

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _grad_pair(fn_gpu, fn_ref, inputs, dtype, tol):
    gi = [t.detach().to("cuda", dtype if t.is_floating_point() else t.dtype).requires_grad_(t.is_floating_point())
          for t in inputs]
    ri = [t.detach().float().requires_grad_() if t.is_floating_point() else t for t in inputs]
    yg, yr = fn_gpu(*gi), fn_ref(*ri)
    assert _rel(yg.cpu(), yr) < tol
    dy = torch.randn_like(yr)
    yg.backward(dy.to("cuda", yg.dtype))
    yr.backward(dy)
    for g, r in zip(gi, ri):
        if r.is_floating_point() and r.grad is not None:
            assert g.grad is not None
            assert _rel(g.grad.cpu(), r.grad) < tol, (g.shape,)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-4)])
@pytest.mark.parametrize("h", [256, 4096, 5120])
@pytest.mark.parametrize("rms", [True, False])
def test_norm(dtype, tol, h, rms):
    torch.manual_seed(0)
    x = torch.randn(37, 3, h) * 2 + 0.5
    w = torch.rand(h) + 0.5
    b = torch.randn(h) * 0.1
    if rms:
        _grad_pair(lambda x, w: core.rmsnorm(x, w, 1e-5), lambda x, w: core._norm_ref(x, w, None, 1e-5, True, False),
                   [x, w], dtype, tol)
    else:
        _grad_pair(lambda x, w, b: core.layernorm(x, w, b, 1e-5),
                   lambda x, w, b: core._norm_ref(x, w, b, 1e-5, False, False), [x, w, b], dtype, tol)


def test_norm_main_grad_accumulates():
    h = 512
    x = torch.randn(64, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.nn.Parameter(torch.ones(h, device="cuda", dtype=torch.bfloat16))
    w.main_grad = torch.zeros(h, device="cuda", dtype=torch.float32)
    for _ in range(2):
        core.rmsnorm(x, w).sum().backward()
    xr = x.detach().float().requires_grad_()
    wr = torch.ones(h, device="cuda", requires_grad=True)
    core._norm_ref(xr, wr, None, 1e-5, True, False).sum().backward()
    assert w.grad is None
    assert _rel(w.main_grad, 2 * wr.grad) < 2e-2


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-5)])
def test_swiglu_and_gelu(dtype, tol):
    torch.manual_seed(1)
    x = torch.randn(50, 2, 1024)
    _grad_pair(core.swiglu, core._swiglu_ref, [x], dtype, tol)
    b = torch.randn(1024) * 0.2
    _grad_pair(core.bias_gelu, core._gelu_ref, [x, b], dtype, tol)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("rot_frac", [1.0, 0.5])
def test_rope(interleaved, rot_frac):
    torch.manual_seed(2)
    s, b, n, hn = 33, 2, 4, 64
    rot = int(hn * rot_frac)
    cos, sin = core.rope_tables(s, rot)
    t = torch.randn(s, b, n, hn)
    _grad_pair(lambda t: core.apply_rope(t, cos.cuda(), sin.cuda(), interleaved),
               lambda t: core._rope_ref(t, cos, sin, interleaved), [t], torch.float32, 1e-5)


def test_rope_qkv_inplace():
    torch.manual_seed(3)
    s, b, ng, qpg, hn = 16, 2, 2, 3, 64
    cos, sin = core.rope_tables(s, hn)
    base = torch.randn(s, b, ng, qpg + 2, hn)
    g = base.clone().cuda().requires_grad_()
    out = core.apply_rope_qkv_(g * 1.0, cos.cuda(), sin.cuda())
    r = base.clone().requires_grad_()
    ref = core.apply_rope_qkv_(r, cos, sin)
    assert _rel(out.cpu(), ref) < 1e-5
    dy = torch.randn_like(ref)
    out.backward(dy.cuda())
    ref.backward(dy)
    assert _rel(g.grad.cpu(), r.grad) < 1e-5


def test_bias_dropout_add():
    torch.manual_seed(4)
    x = torch.randn(128, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(128, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    bias = torch.randn(1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = core.bias_dropout_add(x, bias, res, 0.0, True)
    assert _rel(out, x.float() + bias.float() + res.float()) < 1e-2
    out = core.bias_dropout_add(x, bias, res, 0.25, True, seed=7)
    kept = ((out.float() - res.float()).abs() > 0).float().mean().item()
    assert 0.70 < kept < 0.80
    out.sum().backward()
    assert abs(x.grad.float().mean().item() - 1.0) < 0.05       # E[mask/(1-p)] = 1
    assert torch.all(res.grad == 1)


def test_embedding():
    torch.manual_seed(5)
    w = torch.randn(100, 64)
    idx = torch.randint(0, 200, (7, 9))
    wg = torch.nn.Parameter(w.cuda())
    out = core.embedding(idx.cuda(), wg, 50, 150)
    ref = core.embedding(idx, w.clone().requires_grad_(), 50, 150)
    assert torch.equal(out.cpu(), ref)
    wr = w.clone().requires_grad_()
    core.embedding(idx, wr, 50, 150).sum().backward()
    out.sum().backward()
    assert _rel(wg.grad.cpu(), wr.grad) < 1e-6


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-5)])
@pytest.mark.parametrize("ls", [0.0, 0.1])
@pytest.mark.parametrize("v", [1000, 32000, 1003 * 8])
def test_cross_entropy(dtype, tol, ls, v):
    torch.manual_seed(6)
    rows = 33
    logits = (torch.randn(rows, v) * 3).to(dtype).float()
    tgt = torch.randint(0, v, (rows,))
    lg = logits.cuda().to(dtype).requires_grad_()
    loss = core.cross_entropy(lg, tgt.cuda(), label_smoothing=ls, inplace_backward=False)
    lr = logits.clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy(lr, tgt, reduction="none", label_smoothing=ls)
    assert _rel(loss.cpu(), ref) < 1e-4
    g = torch.rand(rows)
    loss.backward(g.cuda())
    ref.backward(g)
    assert _rel(lg.grad.cpu(), lr.grad) < tol


def test_cross_entropy_vocab_shard_stats_combine():
    """Two shards combined by hand reproduce the full-vocab loss (the cross-rank algebra)."""
    torch.manual_seed(7)
    rows, v = 16, 512
    logits = torch.randn(rows, v, device="cuda") * 4
    tgt = torch.randint(0, v, (rows,), device="cuda")
    ref = torch.nn.functional.cross_entropy(logits, tgt, reduction="none")
    from megatron_lm_b200.ops import _lib
    stats = []
    for r in range(2):
        sh = logits[:, r * 256:(r + 1) * 256].contiguous()
        st = torch.empty(4, rows, device="cuda")
        _lib.check(_lib.lib().mlb_ce_fwd(0, sh.data_ptr(), tgt.data_ptr(), st[0].data_ptr(), st[1].data_ptr(),
                                         st[2].data_ptr(), st[3].data_ptr(), rows, 256, 256, r * 256, _lib.stream()), "ce")
        stats.append(st)
    gmax = torch.maximum(stats[0][0], stats[1][0])
    gsum = sum(s[1] * torch.exp(s[0] - gmax) for s in stats)
    tg = stats[0][2] + stats[1][2]
    assert _rel(torch.log(gsum) + gmax - tg, ref) < 1e-5


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_adam_matches_torch(gdtype):
    torch.manual_seed(8)
    n = 50_000 + 3
    p0 = torch.randn(n)
    segs = [(0, 20_000, 0), (20_000, 64, 1), (20_064, n - 20_064, 0)]
    p = p0.clone().cuda()
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    table, nchunks = optim.build_chunk_table(segs, "cuda")
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([{"params": [ref], "weight_decay": 0.0}], lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for step in range(1, 4):
        g = torch.randn(n).to(gdtype)
        ref.grad = g.float().clone()
        opt.step()
        optim.adam_step(p, m, v, g.cuda(), table=table, nchunks=nchunks, lrs=[1e-2, 1e-2], wds=[0.0, 0.0],
                        beta1=0.9, beta2=0.95, eps=1e-8, step=step, p_lp=lp)
    assert _rel(p.cpu(), ref.detach()) < 1e-5
    assert _rel(lp.cpu(), ref.detach()) < 5e-3
    # weight decay only in group 0, skip flag, grad scale
    p2 = p0.clone().cuda(); m.zero_(); v.zero_()
    skip = torch.ones(1, device="cuda")
    optim.adam_step(p2, m, v, torch.ones(n, device="cuda"), table=table, nchunks=nchunks, lrs=[0.1, 0.1],
                    wds=[0.5, 0.0], beta1=0.9, beta2=0.95, eps=1e-8, step=1, skip=skip)
    assert torch.equal(p2.cpu(), p0)
    optim.adam_step(p2, m, v, torch.ones(n, device="cuda"), table=table, nchunks=nchunks, lrs=[0.1, 0.1],
                    wds=[0.5, 0.0], beta1=0.9, beta2=0.95, eps=1e-8, step=1,
                    grad_scale=torch.full((1,), 2.0, device="cuda"))
    exp = p0.clone()
    exp[:20_000] *= 0.95; exp[20_064:] *= 0.95
    exp -= 0.1
    assert _rel(p2.cpu(), exp) < 1e-5


def test_sumsq_scale_zeros_cast():
    torch.manual_seed(9)
    x = torch.randn(1_000_003, device="cuda")
    assert abs(optim.sum_squares(x).item() / x.double().pow(2).sum().item() - 1) < 1e-5
    a = optim.sum_squares(x); b = optim.sum_squares(x)
    assert torch.equal(a, b)                                   # deterministic
    xb = x.to(torch.bfloat16)
    assert abs(optim.sum_squares(xb).item() / xb.double().pow(2).sum().item() - 1) < 1e-5
    y = x.clone(); optim.scale_(y, 0.5, torch.full((1,), 4.0, device="cuda"))
    assert _rel(y, x * 2) < 1e-6
    z = torch.zeros(1000, device="cuda"); z[::10] = 1
    assert optim.count_zeros(z).item() == 900
    dst = torch.zeros(x.numel(), device="cuda", dtype=torch.bfloat16)
    optim.cast_copy(x, dst)
    assert torch.equal(dst, x.to(torch.bfloat16))
    acc = torch.ones(x.numel(), device="cuda")
    optim.cast_copy(dst, acc, scale=2.0, accumulate=True)
    assert _rel(acc, 1 + 2 * dst.float()) < 1e-6
