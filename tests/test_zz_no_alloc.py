"""The allocation-free norm backward (``mlb_norm_bwd_noalloc``) against the regular entry point.

Some users of the kernel library cannot allocate device memory where they call it - a serving
process running under a frozen memory plan, code that must avoid the device-wide synchronisation
that cudaMalloc / cudaFree can cause in the middle of a step, code running inside another
allocator's hooks.  For them the library keeps the scratch space of the norm backward in a static
device array.  This test calls that entry point through its exported C symbol (plain ctypes, no
helper of the package in between), twice in a row so that the second call runs on a scratch array
still holding the first call's data, and checks it against ``mlb_norm_bwd`` with the tolerance the
other norm tests use.  It lives in a file that pytest collects last, so a run that stops at the
first failure has already run everything else; it also passes when run alone in a fresh process.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "megatron_lm_b200", "_C", "libmlb.so")


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _load():
    lib = ctypes.CDLL(_LIB)
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.mlb_norm_bwd_noalloc.argtypes = [I, I, P, P, P, P, P, P, P, P, I, I, I, I, P]
    lib.mlb_norm_bwd_noalloc.restype = I
    lib.mlb_norm_bwd_noalloc_max_h.argtypes = []
    lib.mlb_norm_bwd_noalloc_max_h.restype = I
    lib.mlb_norm_bwd.argtypes = [I, I, P, P, P, P, P, P, P, P, P, I, I, I, I, P]
    lib.mlb_norm_bwd.restype = I
    lib.mlb_norm_bwd_grid.argtypes = [I]
    lib.mlb_norm_bwd_grid.restype = I
    lib.mlb_norm_fwd.argtypes = [I, I, P, P, P, P, P, P, I, I, ctypes.c_float, I, P]
    lib.mlb_norm_fwd.restype = I
    lib.mlb_set_device.argtypes = [I]
    lib.mlb_set_device.restype = I
    return lib


@pytest.mark.parametrize("rms", [1, 0])
@pytest.mark.parametrize("dtype,code,tol", [(torch.bfloat16, 1, 2e-2), (torch.float32, 0, 1e-4)])
def test_noalloc_matches_regular_entry_point_twice(rms, dtype, code, tol):
    lib = _load()
    assert lib.mlb_set_device(torch.cuda.current_device()) == 0
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(0)
    # later calls reuse the dirty scratch array; the last two are the widest row the array supports, once with
    # fewer rows than the kernel has blocks (most blocks only write zeros) and once with many
    for call, (rows, h) in enumerate([(300, 4096), (77, 1024), (5, 8192), (1500, 8192)]):
        x = (torch.randn(rows, h, device="cuda") * 2 + 0.3).to(dtype)
        dy = torch.randn(rows, h, device="cuda").to(dtype)
        gamma = (torch.rand(h, device="cuda") + 0.5).to(dtype)
        beta = torch.zeros(h, device="cuda", dtype=dtype)
        y = torch.empty_like(x)
        mean = torch.empty(rows, device="cuda")
        rstd = torch.empty(rows, device="cuda")
        assert lib.mlb_norm_fwd(code, rms, x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(),
                                mean.data_ptr(), rstd.data_ptr(), rows, h, 1e-5, 0, stream) == 0
        # regular entry point: caller-allocated workspace
        ws = torch.empty(lib.mlb_norm_bwd_grid(rows) * 2 * h, device="cuda")
        dx_ref = torch.empty_like(x)
        dg_ref = torch.empty(h, device="cuda")
        db_ref = torch.empty(h, device="cuda")
        assert lib.mlb_norm_bwd(code, rms, dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                rstd.data_ptr(), dx_ref.data_ptr(), dg_ref.data_ptr(), db_ref.data_ptr(),
                                ws.data_ptr(), rows, h, 0, 0, stream) == 0
        # allocation-free entry point: outputs only
        dx = torch.empty_like(x)
        dg = torch.empty(h, device="cuda")
        db = torch.empty(h, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = lib.mlb_norm_bwd_noalloc(code, rms, dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                      rstd.data_ptr(), dx.data_ptr(), dg.data_ptr(), db.data_ptr(), rows, h, 0, 0,
                                      stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert _rel(dx, dx_ref) < tol, (call, _rel(dx, dx_ref))
        assert _rel(dg, dg_ref) < tol, (call, _rel(dg, dg_ref))
        if not rms:
            assert _rel(db, db_ref) < tol, (call, _rel(db, db_ref))
        # accumulate mode adds to what is there
        dg2 = dg.clone()
        assert lib.mlb_norm_bwd_noalloc(code, rms, dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                        rstd.data_ptr(), dx.data_ptr(), dg2.data_ptr(), db.data_ptr(), rows, h, 0, 1,
                                        stream) == 0
        torch.cuda.synchronize()
        assert _rel(dg2, 2 * dg_ref) < tol


def test_noalloc_rejects_sizes_beyond_its_array():
    lib = _load()
    assert lib.mlb_set_device(torch.cuda.current_device()) == 0
    max_h = lib.mlb_norm_bwd_noalloc_max_h()
    assert max_h == 8192
    t = torch.zeros(8, device="cuda")
    args = (t.data_ptr(),) * 8
    assert lib.mlb_norm_bwd_noalloc(0, 1, *args, 4, max_h + 8, 0, 0, None) == -20      # too wide
    assert lib.mlb_norm_bwd_noalloc(0, 1, *args, 4, 12, 0, 0, None) == -20             # not a multiple of 8
    assert lib.mlb_norm_bwd_noalloc(0, 1, *args, 0, 64, 0, 0, None) == -20             # no rows
    assert lib.mlb_norm_bwd_noalloc(7, 1, *args, 4, 64, 0, 0, None) == -21             # unknown dtype
