"""Kernel microbenchmarks: ``python -m megatron_lm_b200.ops.microbench <op> [options]``.

Each op is timed with CUDA events on the launching stream after warm-up, with a synchronize on both
sides; operands are sized (or cycled) so that the working set exceeds the 126 MB L2.  Throughput is
printed next to the fraction of the measured machine peaks when a ``MEASURED_PEAKS.json`` (keys
``hbm_gbs``, ``bf16_tflops``) is found in the working directory.  ``--iters`` small (1-3) makes the run
suitable for a profiler capture of a single kernel.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    try:
        with open("MEASURED_PEAKS.json") as f:
            return json.load(f)
    except OSError:
        return {}


_BLOCKER = {}


def _blocker():
    """A product of about a millisecond in front of every timed call: while the GPU works on it the host enqueues the
    call and the closing event, so the events bracket device time only (an op of 50 us issued from Python is otherwise
    timed at the host's launch rate), and its 400 MB of operands push the previous iteration's data out of L2."""
    dev = torch.cuda.current_device()
    if dev not in _BLOCKER:
        a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
        _BLOCKER[dev] = (a, torch.empty_like(a))
    a, out = _BLOCKER[dev]
    torch.matmul(a, a, out=out)


def _time(fn, iters, warmup):
    """Median device time of ``fn`` over ``iters`` calls (the median, because a call whose launch the host delivers
    late - an allocator that has to go to the driver, a collection - leaves the GPU idle inside its interval)."""
    _blocker()                                  # its buffers are allocated outside the timed calls
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for e0, e1 in ev:
        _blocker()
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    t = sorted(e0.elapsed_time(e1) for e0, e1 in ev)
    return t[len(t) // 2]


def _report(name, ms, flops=None, bytes_=None):
    pk = _peaks()
    msg = f"{name}: {ms * 1e3:.1f} us"
    if flops:
        tf = flops / ms / 1e9
        msg += f"  {tf:.0f} TFLOP/s"
        if pk.get("bf16_tflops"):
            msg += f" ({tf / pk['bf16_tflops']:.2f} of measured cuBLAS burst)"
    if bytes_:
        gb = bytes_ / ms / 1e6
        msg += f"  {gb:.0f} GB/s"
        if pk.get("hbm_gbs"):
            msg += f" ({gb / pk['hbm_gbs']:.2f} of measured copy bandwidth)"
    print(msg, flush=True)


def bench_gemm(a):
    from .gemm import gemm
    M, N, K = a.m, a.n, a.k
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    fl = 2.0 * M * N * K
    _report(f"gemm fwd {M}x{N}x{K} bf16", _time(lambda: gemm(A, B, out=out), a.iters, a.warmup), fl)
    if a.all:
        Bt, At = B.t().contiguous(), A.t().contiguous()
        _report("  dgrad form (B MN-major)", _time(lambda: gemm(A, Bt, b_mn=True, out=out), a.iters, a.warmup), fl)
        o32 = torch.zeros(M, N, device="cuda", dtype=torch.float32)
        _report("  wgrad form (A, B MN-major, fp32 accumulate)",
                _time(lambda: gemm(At, Bt, a_mn=True, b_mn=True, out=o32, accumulate=True), a.iters, a.warmup), fl)
        _report("  torch.matmul (cuBLAS)", _time(lambda: torch.matmul(A, B.t(), out=out), a.iters, a.warmup), fl)
    if a.fp8:
        from . import fp8
        qa, qb = fp8.quantize(A, 0, transpose=False), fp8.quantize(B, 0, transpose=False)
        _report("  fp8 e4m3, per-tensor scales", _time(lambda: fp8.gemm_fp8(qa.data, 0, qa.scale_inv, qb.data, 0, qb.scale_inv,
                                                                         out=out), a.iters, a.warmup), fl)
        ma, _ = fp8.mxfp8_quantize_dual(A, colwise=False)
        mb, _ = fp8.mxfp8_quantize_dual(B, colwise=False)
        _report("  mxfp8 (1x32 block scales in the tensor core)", _time(lambda: fp8.gemm_mx(ma, mb, out=out), a.iters, a.warmup), fl)
        _report("  mxfp8 dual quantiser (row-wise + transposed column-wise copy)",
                _time(lambda: fp8.mxfp8_quantize_dual(A), a.iters, a.warmup), bytes_=A.numel() * 4)


def bench_attention(a):
    from .attention import attention_bwd_raw, attention_fwd_raw
    s, b, ng, qpg, d = a.seq, a.batch, a.groups, a.heads // a.groups, a.head_dim
    qkv = torch.randn(s, b, ng, qpg + 2, d, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, :, :, :qpg], qkv[:, :, :, qpg], qkv[:, :, :, qpg + 1]
    scale = d ** -0.5
    fl = 4.0 * s * s * b * a.heads * d * (0.5 if a.causal else 1.0)
    o, lse = attention_fwd_raw(q, k, v, a.causal, scale)
    _report(f"attention fwd s={s} b={b} heads={a.heads} d={d} causal={a.causal}",
            _time(lambda: attention_fwd_raw(q, k, v, a.causal, scale), a.iters, a.warmup), fl)
    do = torch.randn_like(o)
    _report("attention bwd", _time(lambda: attention_bwd_raw(q, k, v, o, do, lse, a.causal, scale), a.iters, a.warmup),
            2.5 * fl)
    if a.library:
        # same-box library bar: torch SDPA on the cuDNN backend (falls back to its flash backend), [b, h, s, d] views
        import torch.nn.functional as F
        from torch.nn.attention import SDPBackend, sdpa_kernel
        ql = q.reshape(s, b, a.heads, d).permute(1, 2, 0, 3).detach().requires_grad_(True)
        kl = k.unsqueeze(3).expand(s, b, ng, qpg, d).reshape(s, b, a.heads, d).permute(1, 2, 0, 3).detach().requires_grad_(True)
        vl = v.unsqueeze(3).expand(s, b, ng, qpg, d).reshape(s, b, a.heads, d).permute(1, 2, 0, 3).detach().requires_grad_(True)
        for name, be in (("cuDNN", SDPBackend.CUDNN_ATTENTION), ("flash", SDPBackend.FLASH_ATTENTION)):
            try:
                with sdpa_kernel([be]):
                    f = lambda: F.scaled_dot_product_attention(ql, kl, vl, is_causal=bool(a.causal), scale=scale)
                    out = f()
                    _report(f"  torch SDPA ({name}) fwd", _time(f, a.iters, a.warmup), fl)
                    gl = torch.randn_like(out)
                    _report(f"  torch SDPA ({name}) bwd",
                            _time(lambda: torch.autograd.grad(out, (ql, kl, vl), gl, retain_graph=True), a.iters, a.warmup),
                            2.5 * fl)
            except Exception as e:       # backend not built into this torch
                print(f"  torch SDPA ({name}): unavailable ({type(e).__name__})", flush=True)


def bench_norm(a):
    from . import core as ops
    x = torch.randn(a.rows, a.hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(a.hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    by = x.numel() * 2 * 2
    _report(f"rmsnorm fwd [{a.rows}, {a.hidden}]", _time(lambda: ops.rmsnorm(x, w, 1e-5, False), a.iters, a.warmup), bytes_=by)
    y = ops.rmsnorm(x, w, 1e-5, False)
    g = torch.randn_like(y)
    _report("rmsnorm bwd", _time(lambda: torch.autograd.grad(y, (x, w), g, retain_graph=True), a.iters, a.warmup),
            bytes_=x.numel() * 2 * 3)


def bench_adam(a):
    from . import optim as kops
    n = a.numel
    p, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    g = torch.randn(n, device="cuda")
    lp = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    segs = [(0, n, 0)]
    table, nc = kops.build_chunk_table(segs, p.device)
    f = lambda: kops.adam_step(p, m, v, g, table=table, nchunks=nc, lrs=[1e-3], wds=[0.1], beta1=0.9, beta2=0.95,
                               eps=1e-8, step=1, p_lp=lp, segments=segs)
    _report(f"adam (fp32 p/m/v + bf16 copy) n={n}", _time(f, a.iters, a.warmup), bytes_=n * (4 * 7 + 2))


def bench_router(a):
    from .router import fused_topk_router
    lg = torch.randn(a.tokens, a.experts, device="cuda", requires_grad=True)
    by = a.tokens * a.experts * (4 + 4 + 1)
    f = lambda: fused_topk_router(lg, a.topk, "softmax_post", None, None, 1e-2, 1e-3)
    _report(f"router fwd T={a.tokens} E={a.experts} k={a.topk}", _time(f, a.iters, a.warmup), bytes_=by)
    probs = f()[0]
    g = torch.randn_like(probs)
    _report("router bwd", _time(lambda: torch.autograd.grad(probs, lg, g, retain_graph=True), a.iters, a.warmup),
            bytes_=a.tokens * a.experts * (4 + 1 + 4 + 4))

    def unfused():
        p = torch.softmax(lg, -1)
        v, i = torch.topk(lg, a.topk, dim=1)
        w = torch.softmax(v, -1)
        dense = torch.zeros_like(lg).scatter(1, i, w)
        m = torch.zeros_like(lg, dtype=torch.bool).scatter(1, i, True)
        return dense, m, m.sum(0), p.sum(0), torch.logsumexp(lg, -1).square().sum()
    _report("router fwd, op-by-op PyTorch", _time(unfused, a.iters, a.warmup))


def bench_sampling(a):
    from .sampling import sample, sample_reference
    lg = torch.randn(a.rows, a.vocab, device="cuda", dtype=torch.bfloat16) * 3
    u = torch.rand(a.rows, device="cuda")
    for name, kw in (("greedy", dict(top_k=1)), ("top-k 50", dict(top_k=50)), ("top-p 0.9", dict(top_p=0.9)),
                     ("multinomial", dict())):
        ms = _time(lambda: sample(lg, u, 0.8, **kw), a.iters, a.warmup)
        ref = _time(lambda: sample_reference(lg, u, 0.8, **kw), max(a.iters // 4, 1), 1)
        _report(f"sample {name} [{a.rows}, {a.vocab}] (sort-based PyTorch: {ref * 1e3:.0f} us)", ms,
                bytes_=lg.numel() * 2)


def bench_gated_norm(a):
    from .mamba import gated_rmsnorm
    y = torch.randn(a.rows, a.hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    z = torch.randn(a.rows, a.hidden, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(a.hidden, device="cuda", requires_grad=True)
    _report(f"gated rmsnorm fwd [{a.rows}, {a.hidden}] groups={a.groups}",
            _time(lambda: gated_rmsnorm(y, z, w, a.groups, 1e-5), a.iters, a.warmup), bytes_=y.numel() * 2 * 3)
    out = gated_rmsnorm(y, z, w, a.groups, 1e-5)
    g = torch.randn_like(out)
    _report("gated rmsnorm bwd", _time(lambda: torch.autograd.grad(out, (y, z, w), g, retain_graph=True), a.iters, a.warmup),
            bytes_=y.numel() * 2 * 5)


def bench_tp_fused(a):
    """Launch with torchrun on tp GPUs of one node.  For the four tensor-parallel products of a transformer layer
    (sizes of the 7B model by default): the GEMM alone, NCCL collective + GEMM as two launches, and the fused
    all-gather->GEMM / GEMM->reduce-scatter kernel; device-timed, max over ranks, against the roofline
    max(FLOPs / GEMM peak, NVLink bytes / 770 GB/s per direction)."""
    import torch.distributed as dist
    from .gemm import gemm
    from .tp_fused import FusedTP
    rank, tp = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    h, f, S = a.hidden, a.ffn, a.seq
    rows = S // tp
    fused = FusedTP(dist.group.WORLD, rows, max(h, 2 * f // tp), max(h, 2 * f // tp))
    pk = _peaks()
    gemm_peak = pk.get("bf16_tflops", 1590.0) * 1e12
    link = 770e9

    def mx(v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def line(name, ms, flops, nv_bytes):
        ms = mx(ms)
        roof = max(flops / gemm_peak, nv_bytes / link) * 1e3
        if rank == 0:
            print(f"  {name}: {ms * 1e3:.1f} us  {flops / ms / 1e9:.0f} TFLOP/s  roofline {roof * 1e3:.1f} us "
                  f"-> {roof / ms:.2f} of roofline", flush=True)
    cases = [("qkv  (all-gather -> GEMM)", "ag", h, 3 * h // tp), ("fc1  (all-gather -> GEMM)", "ag", h, 2 * f // tp),
             ("proj (GEMM -> reduce-scatter)", "rs", h // tp, h), ("fc2  (GEMM -> reduce-scatter)", "rs", f // tp, h)]
    for name, kind, K, N in cases:
        W = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
        flops = 2.0 * S * N * K
        if rank == 0:
            print(f"{name}: M={S} N={N} K={K} tp={tp}", flush=True)
        if kind == "ag":
            x = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
            full = torch.empty(S, K, device="cuda", dtype=torch.bfloat16)
            out = torch.empty(S, N, device="cuda", dtype=torch.bfloat16)
            line("GEMM alone          ", _time(lambda: gemm(full, W, out=out), a.iters, a.warmup), flops, 0)

            def nccl():
                dist.all_gather_into_tensor(full, x)
                gemm(full, W, out=out)
            line("NCCL all-gather+GEMM", _time(nccl, a.iters, a.warmup), flops, (tp - 1) * rows * K * 2)
            line("fused               ", _time(lambda: fused.ag_gemm(x, W), a.iters, a.warmup), flops, (tp - 1) * rows * K * 2)
        else:
            A = torch.randn(S, K, device="cuda").to(torch.bfloat16)
            full = torch.empty(S, N, device="cuda", dtype=torch.bfloat16)
            out = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
            line("GEMM alone          ", _time(lambda: gemm(A, W, out=full), a.iters, a.warmup), flops, 0)

            def nccl():
                gemm(A, W, out=full)
                dist.reduce_scatter_tensor(out, full)
            nv = (tp - 1) * rows * N * 2
            line("GEMM+NCCL red-scat. ", _time(nccl, a.iters, a.warmup), flops, nv)
            line("fused               ", _time(lambda: fused.gemm_rs(A, W), a.iters, a.warmup), flops, nv)
    torch.cuda.synchronize()
    from . import _lib
    _lib.check_status()
    dist.barrier()
    dist.destroy_process_group()


def bench_tcgen05(a):
    """Issue and completion time of batches of 16 ``tcgen05.mma`` instructions on one SM (``csrc/probe.cu``)."""
    from . import _lib
    _lib.register_signatures({"mlb_tcgen05_probe": "ppp"})
    out = torch.zeros(18, dtype=torch.int64, device="cuda")
    _lib.check(_lib.lib().mlb_tcgen05_probe(out.data_ptr(), _lib.status_word().data_ptr(), _lib.stream()), "probe")
    torch.cuda.synchronize()
    v = out.tolist()
    i = 0
    for n in (64, 128, 256):
        for name in ("A, B shared memory", "A tensor memory", "A tensor memory, B MN-major"):
            math = n // 4 * 2                       # 128 x n x 16 at 8192 FLOP per cycle
            print(f"16 x (128 x {n:3d} x 16), {name:28s}: issued in {v[2 * i]:5d} cycles, complete after {v[2 * i + 1]:5d} "
                  f"({v[2 * i + 1] / 16:5.1f} per instruction; arithmetic alone {math})")
            i += 1


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    sub = ap.add_subparsers(dest="op", required=True)
    g = sub.add_parser("gemm"); g.add_argument("--m", type=int, default=8192); g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=8192); g.add_argument("--all", action="store_true")
    g.add_argument("--fp8", action="store_true", help="also time the per-tensor FP8 and the block-scaled MXFP8 kernels")
    t = sub.add_parser("attention"); t.add_argument("--seq", type=int, default=4096); t.add_argument("--batch", type=int, default=4)
    t.add_argument("--heads", type=int, default=32); t.add_argument("--groups", type=int, default=32)
    t.add_argument("--head-dim", type=int, default=128); t.add_argument("--causal", type=int, default=1)
    t.add_argument("--library", action="store_true", help="also time torch SDPA (cuDNN / flash backends) on the same shapes")
    n = sub.add_parser("norm"); n.add_argument("--rows", type=int, default=32768); n.add_argument("--hidden", type=int, default=4096)
    d = sub.add_parser("adam"); d.add_argument("--numel", type=int, default=1 << 28)
    r = sub.add_parser("router"); r.add_argument("--tokens", type=int, default=1 << 20)
    r.add_argument("--experts", type=int, default=64); r.add_argument("--topk", type=int, default=6)
    sp = sub.add_parser("sampling"); sp.add_argument("--rows", type=int, default=512)
    sp.add_argument("--vocab", type=int, default=131072)
    gn = sub.add_parser("gated-norm"); gn.add_argument("--rows", type=int, default=32768)
    gn.add_argument("--hidden", type=int, default=4096); gn.add_argument("--groups", type=int, default=8)
    tf = sub.add_parser("tp-fused", help="torchrun --nproc-per-node TP -m megatron_lm_b200.ops.microbench tp-fused")
    tf.add_argument("--hidden", type=int, default=4096); tf.add_argument("--ffn", type=int, default=11008)
    tf.add_argument("--seq", type=int, default=4096)
    sub.add_parser("tcgen05", help="tensor-core instruction issue / completion times on one SM")
    a = ap.parse_args(argv)
    {"tcgen05": bench_tcgen05, "tp-fused": bench_tp_fused, "gemm": bench_gemm, "attention": bench_attention, "norm": bench_norm, "adam": bench_adam, "router": bench_router,
     "sampling": bench_sampling, "gated-norm": bench_gated_norm}[a.op](a)
    from . import _lib
    _lib.check_status()


if __name__ == "__main__":
    main()
