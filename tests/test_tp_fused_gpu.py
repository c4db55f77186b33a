"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels on 2+ GPUs against NCCL + fp32 matmul,
and a TP+SP model trained with them against the same model on the NCCL path."""
import pytest
import torch

from tests.gpu_dist_utils import run_on_gpus

pytestmark = pytest.mark.gpu


def _n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _kernels(rank, world, rows, K, N):
    import torch.distributed as dist
    from megatron_lm_b200.ops import _lib
    from megatron_lm_b200.ops.tp_fused import FusedTP
    torch.manual_seed(7)
    group = dist.group.WORLD
    f = FusedTP(group, rows, max(K, N), max(K, N))
    dev = torch.device("cuda", rank)
    W = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)          # same on every rank (same seed)
    for call in range(3):                                                     # sequence numbers advance
        torch.manual_seed(100 * call + rank)
        x = torch.randn(rows, K, device=dev).to(torch.bfloat16)
        y, gathered = f.ag_gemm(x, W)
        full = torch.empty(world * rows, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x)
        torch.cuda.synchronize()
        _lib.check_status()
        assert torch.equal(gathered, full), f"call {call}: gathered rows differ"
        assert _rel(y, full.float() @ W.float().t()) < 1e-2
        # dgrad layout (weight stored [K, N] seen as MN-major B)
        y2, _ = f.ag_gemm(x, W.t().contiguous(), b_mn=True)
        assert _rel(y2, full.float() @ W.float().t()) < 1e-2
        # reduce-scatter: every rank multiplies its own A; rows [rank*rows, (rank+1)*rows) come back summed
        torch.manual_seed(1000 * call + rank)
        A = torch.randn(world * rows, K, device=dev).to(torch.bfloat16)
        res = torch.randn(rows, N, device=dev).to(torch.bfloat16)
        out = f.gemm_rs(A, W, residual=res if call == 1 else None)
        ref_full = (A.float() @ W.float().t())
        dist.all_reduce(ref_full)
        ref = ref_full[rank * rows:(rank + 1) * rows]
        if call == 1:
            ref = ref + res.float()
        torch.cuda.synchronize()
        _lib.check_status()
        assert _rel(out, ref) < 1.5e-2, (call, _rel(out, ref))


@pytest.mark.skipif(_n_gpus() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("rows,K,N", [(128, 256, 512), (256, 1024, 768), (1024, 4096, 3072)])
def test_fused_kernels_2gpu(rows, K, N):
    run_on_gpus(_kernels, 2, rows, K, N)


@pytest.mark.skipif(_n_gpus() < 4, reason="needs 4 GPUs")
@pytest.mark.parametrize("rows,K,N", [(256, 1024, 1024), (1024, 4096, 1024), (1024, 2752, 4096)])
def test_fused_kernels_4gpu(rows, K, N):
    # 256-row multiples per rank: the CTA-pair kernel in both communication modes at tp 4
    run_on_gpus(_kernels, 4, rows, K, N)


def _kernels_partly_resident(rank, world, rows, K, N):
    """Part of the GPU is held by another stream's long-running kernel while the fused kernels run: with tiles
    handed to running blocks only, they finish (correctly) long before the holder leaves."""
    import torch.distributed as dist
    from megatron_lm_b200.ops import _lib
    from megatron_lm_b200.ops.tp_fused import FusedTP, occupy_sms
    f = FusedTP(dist.group.WORLD, rows, max(K, N), max(K, N))
    assert f.sched is not None
    dev = torch.device("cuda", rank)
    torch.manual_seed(3)
    W = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    torch.manual_seed(50 + rank)
    x = torch.randn(rows, K, device=dev).to(torch.bfloat16)
    A = torch.randn(world * rows, K, device=dev).to(torch.bfloat16)
    full = torch.empty(world * rows, K, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(full, x)
    ref_full = A.float() @ W.float().t()
    dist.all_reduce(ref_full)
    f.ag_gemm(x, W); f.gemm_rs(A, W)                       # warm-up (module load, first-touch)
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream()
    hold_us = 300000
    # a different number of held SMs on every rank, each too full of shared memory to take a GEMM block
    occupy_sms(24 + 20 * rank, 200 * 1024, hold_us, side)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        y, gathered = f.ag_gemm(x, W)
        out = f.gemm_rs(A, W)
    e1.record()
    torch.cuda.synchronize()
    _lib.check_status()
    assert e0.elapsed_time(e1) < hold_us / 1e3 * 0.5, e0.elapsed_time(e1)      # did not wait for the holders
    assert torch.equal(gathered, full)
    assert _rel(y, full.float() @ W.float().t()) < 1e-2
    assert _rel(out, ref_full[rank * rows:(rank + 1) * rows]) < 1.5e-2


@pytest.mark.skipif(_n_gpus() < 2, reason="needs 2 GPUs")
def test_fused_kernels_with_part_of_the_gpu_held():
    run_on_gpus(_kernels_partly_resident, min(_n_gpus(), 4), 1024, 2048, 2048)


def _model(rank, world, fused, out_path):
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.ops import _lib
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.training.training import setup_model_and_optimizer, train_step
    from tests.model_utils import reinit_by_global_name
    state.initialize_model_parallel(tensor_model_parallel_size=world, create_gloo_process_groups=False)
    V, S, B = 1024, 512, 1
    cfg = TransformerConfig(num_layers=2, hidden_size=512, num_attention_heads=8, ffn_hidden_size=1024,
                            normalization="RMSNorm", gated_linear_unit=True, activation_func="silu",
                            add_bias_linear=False, hidden_dropout=0.0, attention_dropout=0.0, bf16=True,
                            params_dtype=torch.bfloat16, tensor_model_parallel_size=world, sequence_parallel=True,
                            kv_channels=64, tp_comm_overlap=fused)

    def provider(pre_process=True, post_process=True, vp_stage=None):
        m = GPTModel(cfg, V, S, position_embedding_type="rope")
        reinit_by_global_name(m, cfg, std=0.02)
        return m
    model, opt, _ = setup_model_and_optimizer(provider, cfg, OptimizerConfig(lr=1e-3, clip_grad=1.0, bf16=True),
                                              DistributedDataParallelConfig(grad_reduce_in_fp32=True))
    if fused:
        from megatron_lm_b200.ops.tp_fused import attach_fused_tp
        assert attach_fused_tp(model, cfg, S, B) is not None
    g = torch.Generator().manual_seed(11)
    data = torch.randint(0, V, (4, B, S + 1), generator=g).cuda()
    losses = []
    for step in range(4):
        def fwd(it, m):
            out = m(data[step][:, :-1], labels=data[step][:, 1:])
            return out, (lambda o: (o.float().mean(), {"lm loss": o.float().mean().detach()}))
        l, _, gn, _ = train_step(fwd, None, model, opt, None, cfg, num_microbatches=1, seq_length=S, micro_batch_size=B)
        losses.append((float(l["lm loss"]), float(gn)))
    torch.cuda.synchronize()
    _lib.check_status()
    if rank == 0:
        torch.save(losses, out_path)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs 2 GPUs")
def test_tp_sp_model_fused_matches_nccl_path(tmp_path):
    a, b = str(tmp_path / "nccl.pt"), str(tmp_path / "fused.pt")
    run_on_gpus(_model, 2, False, a)
    run_on_gpus(_model, 2, True, b)
    ta, tb = torch.load(a), torch.load(b)
    for (la, ga), (lb, gb) in zip(ta, tb):
        assert abs(la - lb) < 3e-2, (ta, tb)
        assert abs(ga - gb) < 5e-2 * max(1.0, ga), (ta, tb)
