"""GPU erasure-coded checkpoint over symmetric memory on 2-4 GPUs: byte-exact rebuild of lost ranks,
parity equal to the CPU oracle."""
import numpy as np
import pytest
import torch

from tests.gpu_dist_utils import run_on_gpus

pytestmark = pytest.mark.gpu


def _worker(rank, world, k, m, lose):
    import torch.distributed as dist
    from megatron_lm_b200.checkpoint import gf256
    from megatron_lm_b200.checkpoint.ec_gpu import GpuECCheckpoint
    chunk = 1 << 16
    nbytes = chunk * 5 + 4096                      # not a whole number of chunks
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    a = torch.randint(0, 255, (nbytes - 1024,), dtype=torch.uint8, device="cuda", generator=g)
    b = torch.randn(256, device="cuda", generator=g)                     # 1024 bytes, another dtype
    mgr = GpuECCheckpoint(dist.group.WORLD, nbytes, k=k, m=m, chunk_bytes=chunk)
    mgr.save([a, b], 5)
    mgr.wait()
    # parity 0 of the first stripe this rank owns equals the oracle
    every = [torch.empty_like(mgr.buf) for _ in range(world)]
    dist.all_gather(every, mgr.buf)
    for s in mgr.plan.stripes:
        if s.parity_owners[0] == rank:
            srcs = [every[r][c * chunk:(c + 1) * chunk].cpu().numpy() for r, c in s.data]
            ref = gf256.apply_matrix_numpy(mgr.G[:, :len(srcs)], srcs)
            off = mgr.parity_off + mgr.slot[(s.index, 0)] * chunk
            assert np.array_equal(mgr.buf[off:off + chunk].cpu().numpy(), ref[0])
            break
    ra, rb = a.clone(), b.clone()
    lost = list(range(world - lose, world))
    a.add_(1); b.mul_(2)                            # training moved on; recovery rolls everyone back
    if rank in lost:
        mgr.drop_device_state()
    it = mgr.recover(lost, [a, b])
    assert it == 5 and torch.equal(a, ra) and torch.equal(b, rb)
    # host tier: wipe the device copy and refill from pinned memory
    mgr.drop_device_state()
    mgr.restore_from_host()
    a.zero_()
    mgr.recover([], [a, b])
    assert torch.equal(a, ra)


@pytest.mark.parametrize("world,k,m,lose", [(2, 1, 1, 1), (4, 2, 2, 2), (4, 3, 1, 1)])
def test_gpu_ec_rebuild(world, k, m, lose):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_on_gpus(_worker, world, k, m, lose)


def _overlap_worker(rank, world):
    """Two overlapped saves back to back while the 'training' tensors keep changing: the second save must not
    overwrite the snapshot that the first one's parity kernel still reads, and recovery returns the second snapshot."""
    import torch.distributed as dist
    from megatron_lm_b200.checkpoint.ec_gpu import GpuECCheckpoint
    chunk = 1 << 16
    n = chunk * 40
    g = torch.Generator(device="cuda").manual_seed(11 + rank)
    a = torch.randint(0, 255, (n,), dtype=torch.uint8, device="cuda", generator=g)
    mgr = GpuECCheckpoint(dist.group.WORLD, n, k=world - 1, m=1, chunk_bytes=chunk)
    mgr.save([a], 5, overlap=True)
    a.add_(3)                                       # the step after the save
    keep = a.clone()
    st = mgr.save([a], 6, overlap=True)
    assert "bytes" in st
    a.add_(1)
    if rank == world - 1:
        mgr.drop_device_state()                     # joins the side stream first: the peers' parity kernels read this rank
    it = mgr.recover([world - 1], [a])
    assert it == 6 and torch.equal(a, keep)
    st = mgr.save([a], 7, overlap=True)             # the device times of save 6 are known by now
    mgr.wait()
    assert st.get("encode_ms", 0.0) > 0.0 and int(st.get("of_iteration", -1)) == 6


def test_gpu_ec_overlapped_saves():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_on_gpus(_overlap_worker, 2)
