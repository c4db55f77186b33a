"""Context-parallel attention on GPUs (NCCL transfers around the flash kernels) against one full-sequence call:
ring (p2p), all-gather, Ulysses (a2a) on 2 GPUs, hierarchical a2a+p2p on 4."""
import math

import pytest
import torch

from tests.gpu_dist_utils import run_on_gpus

pytestmark = pytest.mark.gpu


def _n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(rank, world, kind):
    from megatron_lm_b200.ops import _lib
    from megatron_lm_b200.ops.attention import attention
    from megatron_lm_b200.parallel import state
    from megatron_lm_b200.parallel.context_parallel import context_parallel_attention, zigzag_indices
    state.initialize_model_parallel(context_parallel_size=world, create_gloo_process_groups=False,
                                    hierarchical_context_parallel_sizes=[2, world // 2] if kind == "a2a+p2p" else None)
    torch.manual_seed(3)                                  # same tensors on every rank
    S, b, ng, qpg, d = 512 * world, 1, 4, 2, 128
    dev = torch.device("cuda", rank)
    q = torch.randn(S, b, ng, qpg, d, device=dev).to(torch.bfloat16)
    k = torch.randn(S, b, ng, d, device=dev).to(torch.bfloat16)
    v = torch.randn(S, b, ng, d, device=dev).to(torch.bfloat16)
    do = torch.randn(S, b, ng * qpg, d, device=dev).to(torch.bfloat16)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    ref = attention(qr, kr, vr, True, 1 / math.sqrt(d))
    ref.backward(do)
    idx = zigzag_indices(S, world, rank, dev)
    ql, kl, vl = (t[idx].clone().requires_grad_() for t in (q, k, v))
    out = context_parallel_attention(ql, kl, vl, kind, state.get_context_parallel_group())
    out.backward(do[idx])
    torch.cuda.synchronize()
    _lib.check_status()

    def rel(a, b_):
        return ((a.float() - b_.float()).norm() / (b_.float().norm() + 1e-12)).item()
    assert rel(out, ref[idx]) < 2e-2, (kind, rel(out, ref[idx]))
    assert rel(ql.grad, qr.grad[idx]) < 3e-2 and rel(kl.grad, kr.grad[idx]) < 3e-2 and rel(vl.grad, vr.grad[idx]) < 3e-2


@pytest.mark.skipif(_n_gpus() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("kind", ["p2p", "all_gather", "a2a"])
def test_context_parallel_attention_2gpu(kind):
    run_on_gpus(_run, 2, kind)


@pytest.mark.skipif(_n_gpus() < 4, reason="needs 4 GPUs")
def test_hierarchical_context_parallel_attention_4gpu():
    run_on_gpus(_run, 4, "a2a+p2p")
