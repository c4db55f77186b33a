"""State-space ops: depthwise causal conv1d (+SiLU) and the Mamba-2 selective scan.

* ``causal_conv1d(x, w, bias, silu)``: x [b, l, c] channel-last.  CUDA forward/backward kernels
  (``csrc/mamba.cu``); CPU tensors use ``torch.nn.functional.conv1d``.
* ``ssd_scan(...)``: the recurrence h_t = exp(dt A) h + dt x (x) B, y = h C + D x.  Training uses the
  chunked ("state-space dual") formulation written with matmuls so autograd applies; forward-only CUDA
  calls (evaluation, decoding with a carried state) run the recurrence kernel.
  Reference call sites: megatron/core/ssm/mamba_mixer.py:426-530 (training) and :549-700 (step).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

_lib.register_signatures({
    "mlb_causal_conv1d_fwd": "ippppp" "iiiii" "p",
    "mlb_causal_conv1d_bwd": "ippppp" "ppp" "iiiii" "p",
    "mlb_ssd_scan_fwd": "ippppp" "pppp" "iiiiii" "i" "p",
    "mlb_gated_rmsnorm_fwd": "ippppp" "iii" "qq" "f" "p",
    "mlb_gated_rmsnorm_bwd": "ippppp" "ppp" "iii" "qqqq" "p",
})


def _conv_ref(x, w, bias, silu, init=None):
    b, l, c = x.shape
    k = w.shape[1]
    xt = x.transpose(1, 2).float()
    if init is not None:
        xt = torch.cat((init.transpose(1, 2).float(), xt), dim=2)
    else:
        xt = F.pad(xt, (k - 1, 0))
    y = F.conv1d(xt, w.float().unsqueeze(1), None if bias is None else bias.float(), groups=c)
    if silu:
        y = F.silu(y)
    return y.transpose(1, 2).to(x.dtype)


class _ConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, silu):
        xc = x.contiguous()
        b, l, c = xc.shape
        wf = w.float().contiguous()
        bf = None if bias is None else bias.float().contiguous()
        y = torch.empty_like(xc)
        _lib.check(_lib.lib().mlb_causal_conv1d_fwd(_lib.dt(xc), xc.data_ptr(), wf.data_ptr(), _lib.ptr(bf), None,
                                                    y.data_ptr(), b, l, c, w.shape[1], int(silu), _lib.stream()), "conv1d")
        ctx.save_for_backward(xc, wf, bf if bf is not None else torch.empty(0, device=x.device))
        ctx.silu, ctx.has_bias, ctx.wdt, ctx.bdt = silu, bias is not None, w.dtype, None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, wf, bf = ctx.saved_tensors
        b, l, c = xc.shape
        dyc = dy.contiguous()
        g = torch.empty(b, l, c, dtype=torch.float32, device=xc.device)
        dx = torch.empty_like(xc)
        dw = torch.zeros_like(wf)
        db = torch.zeros(c, dtype=torch.float32, device=xc.device) if ctx.has_bias else None
        _lib.check(_lib.lib().mlb_causal_conv1d_bwd(_lib.dt(xc), xc.data_ptr(), wf.data_ptr(),
                                                    bf.data_ptr() if ctx.has_bias else None, dyc.data_ptr(),
                                                    g.data_ptr(), dx.data_ptr(), dw.data_ptr(), _lib.ptr(db), b, l, c,
                                                    wf.shape[1], int(ctx.silu), _lib.stream()), "conv1d_bwd")
        return dx, dw.to(ctx.wdt), None if db is None else db.to(ctx.bdt), None


def causal_conv1d(x, weight, bias=None, silu: bool = True):
    """x [b, l, c], weight [c, k]: y[t] = act(bias + sum_j w[j] x[t-(k-1)+j])."""
    if not x.is_cuda:
        return _conv_ref(x, weight, bias, silu)
    return _ConvFn.apply(x, weight, bias, silu)


def causal_conv1d_update(x_t, conv_state, weight, bias=None, silu: bool = True):
    """One decoding step: x_t [b, c]; conv_state [b, k-1, c] holds the previous inputs and is updated."""
    win = torch.cat((conv_state, x_t.unsqueeze(1)), dim=1)                  # [b, k, c]
    y = (win.float() * weight.float().t().unsqueeze(0)).sum(dim=1)
    if bias is not None:
        y = y + bias.float()
    if silu:
        y = F.silu(y)
    conv_state.copy_(win[:, 1:])
    return y.to(x_t.dtype)


def _segsum(a):
    """a [..., T] -> [..., T, T] with out[i, j] = sum_{j < k <= i} a[k] for i >= j, -inf above the diagonal."""
    T = a.shape[-1]
    cs = torch.cumsum(a, dim=-1)
    out = cs.unsqueeze(-1) - cs.unsqueeze(-2)
    mask = torch.ones(T, T, dtype=torch.bool, device=a.device).tril(0)
    return out.masked_fill(~mask, float("-inf"))


def ssd_chunked(x, dt, A, Bm, Cm, D=None, chunk: int = 64, initial_state=None):
    """Chunked state-space-dual evaluation (fp32).  x [b,l,H,P], dt [b,l,H], A [H], B/C [b,l,G,N].
    Returns (y [b,l,H,P], final_state [b,H,P,N])."""
    b, l, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    pad = (-l) % chunk
    xf, dtf = x.float(), dt.float()
    Bf = Bm.float().repeat_interleave(H // G, dim=2)
    Cf = Cm.float().repeat_interleave(H // G, dim=2)
    if pad:
        xf, dtf = F.pad(xf, (0, 0, 0, 0, 0, pad)), F.pad(dtf, (0, 0, 0, pad))
        Bf, Cf = F.pad(Bf, (0, 0, 0, 0, 0, pad)), F.pad(Cf, (0, 0, 0, 0, 0, pad))
    nc = (l + pad) // chunk
    xd = (xf * dtf.unsqueeze(-1)).view(b, nc, chunk, H, P)
    a = (dtf * A.float()).view(b, nc, chunk, H).permute(0, 3, 1, 2)          # [b,H,nc,T]
    Bc, Cc = Bf.view(b, nc, chunk, H, N), Cf.view(b, nc, chunk, H, N)
    a_cs = torch.cumsum(a, dim=-1)
    Lmat = torch.exp(_segsum(a))                                             # [b,H,nc,T,T]
    y_diag = torch.einsum("bclhn,bcshn,bhcls,bcshp->bclhp", Cc, Bc, Lmat, xd)
    decay_states = torch.exp(a_cs[..., -1:] - a_cs)                          # [b,H,nc,T]
    states = torch.einsum("bclhn,bhcl,bclhp->bchpn", Bc, decay_states, xd)
    init = torch.zeros(b, 1, H, P, N, dtype=torch.float32, device=x.device) if initial_state is None \
        else initial_state.float().unsqueeze(1)
    states = torch.cat((init, states), dim=1)                                # [b,nc+1,H,P,N]
    chunk_decay = torch.exp(_segsum(F.pad(a_cs[..., -1], (1, 0))))           # [b,H,nc+1,nc+1]
    new_states = torch.einsum("bhzc,bchpn->bzhpn", chunk_decay, states)
    prev, final = new_states[:, :-1], new_states[:, -1]
    y_off = torch.einsum("bclhn,bchpn,bhcl->bclhp", Cc, prev, torch.exp(a_cs))
    y = (y_diag + y_off).reshape(b, nc * chunk, H, P)[:, :l]
    if D is not None:
        y = y + x.float() * D.float().view(1, 1, H, 1)
    return y, final


def ssd_scan(x, dt, A, Bm, Cm, D=None, z=None, state: Optional[torch.Tensor] = None, has_init: bool = False,
             chunk: int = 64):
    """Selective scan.  ``state`` (fp32 [b,H,P,N]), when given, supplies the initial state if ``has_init``
    and receives the final one.  ``z`` gates the output with silu(z).  Output has x's dtype."""
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (x, dt, A, Bm, Cm, D, z))
    if x.is_cuda and not needs_grad:
        xc, Bc, Cc = x.contiguous(), Bm.contiguous(), Cm.contiguous()
        b, l, H, P = xc.shape
        G, N = Bc.shape[2], Bc.shape[3]
        dtf = dt.float().contiguous()
        Af = A.float().contiguous()
        Df = None if D is None else D.float().contiguous()
        zc = None if z is None else z.contiguous()
        y = torch.empty_like(xc)
        rc = _lib.lib().mlb_ssd_scan_fwd(_lib.dt(xc), xc.data_ptr(), dtf.data_ptr(), Af.data_ptr(), Bc.data_ptr(),
                                         Cc.data_ptr(), _lib.ptr(Df), _lib.ptr(zc), y.data_ptr(), _lib.ptr(state), b, l,
                                         H, P, G, N, int(has_init), _lib.stream())
        if rc != -5:                       # -5: shape outside the kernel's tiling, use the chunked form below
            _lib.check(rc, "ssd_scan")
            return y
    y, final = ssd_chunked(x, dt, A, Bm, Cm, D, chunk, state if has_init else None)
    if state is not None:
        state.copy_(final)
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(x.dtype)


def ssd_reference(x, dt, A, Bm, Cm, D=None, initial_state=None):
    """Step-by-step recurrence in fp32 (test oracle)."""
    b, l, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    h = torch.zeros(b, H, P, N, dtype=torch.float32, device=x.device) if initial_state is None else initial_state.float().clone()
    Bf = Bm.float().repeat_interleave(H // G, dim=2)
    Cf = Cm.float().repeat_interleave(H // G, dim=2)
    ys = []
    for t in range(l):
        decay = torch.exp(dt[:, t].float() * A.float()).view(b, H, 1, 1)
        h = h * decay + (x[:, t].float() * dt[:, t].float().unsqueeze(-1)).unsqueeze(-1) * Bf[:, t].unsqueeze(2)
        yt = (h * Cf[:, t].unsqueeze(2)).sum(-1)
        if D is not None:
            yt = yt + x[:, t].float() * D.float().view(1, H, 1)
        ys.append(yt)
    return torch.stack(ys, dim=1), h


# ----------------------------------------------------------------------------- gated group RMSNorm
def _gated_rmsnorm_ref(y, z, w, groups, eps):
    u = y.float() * F.silu(z.float())
    shp = u.shape
    ug = u.view(*shp[:-1], groups, shp[-1] // groups)
    ug = ug * torch.rsqrt(ug.pow(2).mean(-1, keepdim=True) + eps)
    return (ug.view(shp) * w.float()).to(y.dtype)


def _rows_view(t, C):
    """[.., C] -> ([rows, C] sharing storage when the rows are evenly strided, else a copy; row stride)."""
    t2 = t.reshape(-1, C)                      # a view whenever the leading dims collapse
    if t2.stride(1) != 1 or t2.stride(0) % 8 != 0 or t2.data_ptr() % 16 != 0:
        t2 = t2.contiguous()
    return t2, t2.stride(0)


class _GatedNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, z, w, groups, eps):
        C = y.shape[-1]
        y2, ys = _rows_view(y, C)
        z2, zs = _rows_view(z, C)
        rows = y2.shape[0]
        wf = w.float().contiguous()
        out = torch.empty(rows, C, dtype=y.dtype, device=y.device)
        rstd = torch.empty(rows, groups, dtype=torch.float32, device=y.device)
        _lib.check(_lib.lib().mlb_gated_rmsnorm_fwd(_lib.dt(y2), y2.data_ptr(), z2.data_ptr(), wf.data_ptr(),
                                                    out.data_ptr(), rstd.data_ptr(), rows, C, groups, ys, zs,
                                                    float(eps), _lib.stream()), "gated_rmsnorm_fwd")
        ctx.save_for_backward(y2, z2, wf, rstd)
        ctx.meta = (groups, y.shape, z.shape, w.dtype)
        return out.view(y.shape)

    @staticmethod
    def backward(ctx, dout):
        y2, z2, wf, rstd = ctx.saved_tensors
        groups, yshape, zshape, wdt = ctx.meta
        rows, C = y2.shape
        do = dout.reshape(rows, C).contiguous()
        dy = torch.empty(rows, C, dtype=y2.dtype, device=y2.device)
        dz = torch.empty(rows, C, dtype=y2.dtype, device=y2.device)
        dw = torch.zeros(C, dtype=torch.float32, device=y2.device)
        _lib.check(_lib.lib().mlb_gated_rmsnorm_bwd(_lib.dt(y2), do.data_ptr(), y2.data_ptr(), z2.data_ptr(),
                                                    wf.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dz.data_ptr(),
                                                    dw.data_ptr(), rows, C, groups, y2.stride(0), z2.stride(0), C, C,
                                                    _lib.stream()), "gated_rmsnorm_bwd")
        return dy.view(yshape), dz.view(zshape), dw.to(wdt), None, None


def gated_rmsnorm(y, z, w, groups: int = 1, eps: float = 1e-5):
    """rmsnorm(y * silu(z)) * w with the mean square over each of ``groups`` contiguous channel groups.
    ``z`` may be a strided slice (same dtype as ``y``).  CUDA kernel for up to 16384 channels and 64 groups with
    group size a multiple of 8; other shapes and CPU tensors use the PyTorch body."""
    C = y.shape[-1]
    ok = (y.is_cuda and z.dtype == y.dtype and y.dtype in (torch.float32, torch.bfloat16, torch.float16)
          and C % 8 == 0 and C <= 16384 and 1 <= groups <= 64 and C % groups == 0 and (C // groups) % 8 == 0)
    if not ok:
        return _gated_rmsnorm_ref(y, z, w, groups, eps)
    return _GatedNormFn.apply(y, z, w, groups, eps)
