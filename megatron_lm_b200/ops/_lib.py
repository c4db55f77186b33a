"""Build and load the native CUDA library (``libmlb.so``).

The kernels are plain ``extern "C"`` entry points that take raw device pointers
and a stream, so the library has no dependency on the PyTorch C++ headers and
compiles in seconds per file.  It is built in-tree for sm_100a only and loaded
with ctypes; an op that runs on a CUDA tensor raises if the library is missing -
there is no silent fallback to another implementation.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.normpath(os.path.join(_HERE, "..", "csrc"))
LIB_DIR = os.path.normpath(os.path.join(_HERE, "..", "_C"))
LIB_PATH = os.path.join(LIB_DIR, "libmlb.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# argument kinds: i int32, l long, p pointer, f float, Q uint64, q int64
_SIGS: Dict[str, str] = {
    "mlb_norm_bwd_grid": "i",
    "mlb_norm_fwd": "iipppppp" "iifip",
    "mlb_norm_bwd": "iippppppppp" "iiiip",
    "mlb_swiglu_fwd": "ipplip",
    "mlb_swiglu_bwd": "ippplip",
    "mlb_bias_gelu_fwd": "ippplip",
    "mlb_bias_gelu_bwd": "ipppplip",
    "mlb_colsum_parts": "l",
    "mlb_colsum": "ippplii" "p",
    "mlb_rope": "ipppp" "iiiiiii" "f" "llllllll" "p",
    "mlb_bias_dropout_add": "ipppppli" "fQQp",
    "mlb_dropout_bwd": "ippplfp",
    "mlb_embedding_fwd": "ippplipp",   # v0/v1 passed as int64 via 'q' below (patched)
    "mlb_embedding_bwd": "ippplipp",
    "mlb_cast": "iipplfip",
    "mlb_ce_fwd": "ipppppp" "lilqp",
    "mlb_ce_fwd_peer": "ipppppp" "lilq" "piil" "p",
    "mlb_ce_combine": "pillfi" "ppp" "p",
    "mlb_ce_bwd": "ippppp" "p" "lilqfip",
    "mlb_adam": "ippppppi" "ppi" "fffff" "ppp",
    "mlb_adam_push": "pppppp" "i" "pi" "ppi" "fffff" "ppp",
    "mlb_grad_pull": "pipl" "f" "pp" "i" "p",
    "mlb_grad_pull_when_ready": "pipl" "f" "p" "pi" "i" "i" "pp",
    "mlb_peer_signal": "piip",
    "mlb_sgd": "ipppppi" "ppi" "fi" "ppp",
    "mlb_sumsq_parts": "",
    "mlb_sumsq": "iplppip",
    "mlb_scale": "iplpfp",
    "mlb_count_zeros": "iplpp",
    "mlb_gemm": "iplipliplipiiiipp",
    "mlb_gemm_pair": "iplipliplipiiiippp",
    "mlb_set_device": "i",
    "mlb_device_sm_count": "i",
}
_SIGS["mlb_embedding_fwd"] = "ippp" "li" "qq" "p"
_SIGS["mlb_embedding_bwd"] = "ippp" "li" "qq" "p"

_CT = {"i": ctypes.c_int, "l": ctypes.c_long, "p": ctypes.c_void_p, "f": ctypes.c_float,
       "Q": ctypes.c_uint64, "q": ctypes.c_int64}

_lib: Optional[ctypes.CDLL] = None


def register_signatures(sigs: Dict[str, str]) -> None:
    """Other op modules add their entry points here before the first load."""
    _SIGS.update(sigs)
    if _lib is not None:
        _bind(_lib, sigs)


def _sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    for f in os.listdir(CSRC):
        if os.path.getmtime(os.path.join(CSRC, f)) > t:
            return True
    return False


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``_C/libmlb.so``."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    os.makedirs(LIB_DIR, exist_ok=True)
    objdir = os.path.join(LIB_DIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdr_time = max([os.path.getmtime(h) for h in headers] + [0.0])

    def compile_one(src: str) -> str:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), hdr_time):
            return obj
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-I", CSRC, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    cmd = [nvcc, "-shared", "-o", LIB_PATH] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


def _bind(lib: ctypes.CDLL, sigs: Dict[str, str]) -> None:
    for name, sig in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise RuntimeError(f"native library lacks symbol {name}; rebuild with build(force=True)") from e
        fn.argtypes = [_CT[c] for c in sig]
        fn.restype = ctypes.c_int


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                "(the CUDA ops of this package have no fallback implementation)")
        _lib = ctypes.CDLL(LIB_PATH)
        _bind(_lib, _SIGS)
    return _lib


def available() -> bool:
    return os.path.exists(LIB_PATH)


_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def dt(t) -> int:
    d = t if isinstance(t, torch.dtype) else t.dtype
    try:
        return _DT[d]
    except KeyError:
        raise TypeError(f"unsupported dtype {d} for a CUDA op of this library")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_tls = threading.local()


# torch.cuda.current_stream() / current_device() go through several Python layers (device-index parsing, lazy-init and
# availability checks, a Stream object) - about 15 us per call, which with one call per kernel launch was a quarter of
# the host's time per training step.  The two built-ins below return the same answers in a fraction of a microsecond.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def device_index() -> int:
    return _raw_device() if _raw_device is not None else torch.cuda.current_device()


def stream() -> int:
    """Current stream handle; also binds this host thread of the library's CUDA runtime to
    the current device the first time the thread calls in (autograd worker threads start
    with no device bound)."""
    dev = device_index()
    if getattr(_tls, "dev", None) != dev:
        torch.cuda.current_device()                   # makes sure the CUDA context of this process exists
        check(lib().mlb_set_device(dev), "set_device")
        _tls.dev = dev
    if _raw_stream is not None:
        return _raw_stream(dev)
    return torch.cuda.current_stream().cuda_stream


launch_count = 0          # kernels of this library launched so far (a caller may reset it)
_KERNELS_PER_CALL = {"norm_bwd": 2, "colsum": 2, "sumsq": 2, "attn_bwd": 3, "set_device": 0}


def check(rc: int, what: str) -> None:
    global launch_count
    launch_count += _KERNELS_PER_CALL.get(what, 1)
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}"
                           + (" (CUDA error)" if rc > 0 else " (argument/shape not supported)"))


_status: Dict[int, torch.Tensor] = {}


def status_word() -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write a non-zero code to when a
    wait ran out.  Read it with :func:`check_status` at a point where a sync is acceptable."""
    d = device_index()
    t = _status.get(d)
    if t is None:
        t = _status[d] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{d}")
    return t


def check_status() -> None:
    code = int(status_word().item())
    if code != 0:
        status_word().zero_()
        raise RuntimeError(f"a device-side wait timed out (code {code}); results of the last step are invalid")
