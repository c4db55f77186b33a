"""GF(2^8) encode / decode kernel against the table-lookup CPU oracle (byte exact)."""
import itertools

import numpy as np
import pytest
import torch

from megatron_lm_b200.checkpoint import gf256
from megatron_lm_b200.ops.ec import ec_apply

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("k,m", [(2, 1), (6, 2), (8, 4), (16, 3)])
def test_encode_matches_oracle_and_decodes(k, m):
    torch.manual_seed(0)
    n = 1 << 20
    data = [torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda") for _ in range(k)]
    G = gf256.generator_matrix(k, m)
    parity = [torch.empty(n, dtype=torch.uint8, device="cuda") for _ in range(m)]
    ec_apply(G, data, parity, n)
    ref = gf256.apply_matrix_numpy(G, [d.cpu().numpy() for d in data])
    for p, r in zip(parity, ref):
        assert np.array_equal(p.cpu().numpy(), r)
    members = data + parity
    lost = list(range(m))                                   # lose the first m data members
    present = [i for i in range(k + m) if i not in lost]
    M, use = gf256.decode_matrix(k, m, present, lost)
    rebuilt = [torch.empty(n, dtype=torch.uint8, device="cuda") for _ in lost]
    ec_apply(M, [members[u] for u in use], rebuilt, n)
    for w, r in zip(lost, rebuilt):
        assert torch.equal(r, members[w])


def test_raw_pointers_and_cpu_path_agree():
    n = 4096
    a = torch.randint(0, 256, (n,), dtype=torch.uint8)
    b = torch.randint(0, 256, (n,), dtype=torch.uint8)
    G = gf256.generator_matrix(2, 2)
    out_cpu = [torch.empty(n, dtype=torch.uint8) for _ in range(2)]
    ec_apply(G, [a, b], out_cpu, n)
    ag, bg = a.cuda(), b.cuda()
    out_gpu = [torch.empty(n, dtype=torch.uint8, device="cuda") for _ in range(2)]
    ec_apply(G, [ag.data_ptr(), bg.data_ptr()], out_gpu, n)
    for c, g in zip(out_cpu, out_gpu):
        assert torch.equal(c, g.cpu())


@pytest.mark.parametrize("k,m,n_jobs", [(6, 2, 5), (2, 2, 3), (16, 4, 2), (1, 1, 4)])
def test_staged_batch_kernel_matches_oracle(k, m, n_jobs):
    """The batched kernel that stages its sources in shared memory with bulk copies (the form used across GPUs),
    on local buffers: every job's parities must equal the table-lookup oracle byte for byte."""
    from megatron_lm_b200.checkpoint.ec_gpu import _JOB
    from megatron_lm_b200.ops import _lib
    torch.manual_seed(1)
    nbytes = 64 * 1024
    G = gf256.generator_matrix(k, m)
    data = [[torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(k)] for _ in range(n_jobs)]
    par = [[torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(m)] for _ in range(n_jobs)]
    jobs = np.zeros(n_jobs, dtype=_JOB)
    for j in range(n_jobs):
        for pos in range(k):
            jobs[j]["src"][pos] = data[j][pos].data_ptr()
            for i in range(m):
                jobs[j]["coef"][i][pos] = G[i, pos]
        for i in range(m):
            jobs[j]["dst"][i] = par[j][i].data_ptr()
        jobs[j]["k"], jobs[j]["m"] = k, m
    tbl = torch.from_numpy(jobs.view(np.uint8).reshape(-1).copy()).cuda()
    st = _lib.status_word()
    for blocks in (0, 3):                                    # whole GPU, and a capped grid
        for p in itertools.chain.from_iterable(par):
            p.zero_()
        _lib.check(_lib.lib().mlb_ec_apply_batch_staged(tbl.data_ptr(), n_jobs, nbytes, k, blocks, st.data_ptr(),
                                                        torch.cuda.current_stream().cuda_stream), "ec staged")
        torch.cuda.synchronize()
        _lib.check_status()
        for j in range(n_jobs):
            ref = gf256.apply_matrix_numpy(G, [d.cpu().numpy() for d in data[j]])
            for p, r in zip(par[j], ref):
                assert np.array_equal(p.cpu().numpy(), r), (j, blocks)
