"""Post-training quantisation of the tensor-parallel linears: calibrate, simulate, compress.

The reference delegates this to an external library (nvidia-modelopt) behind
megatron/post_training/arguments.py:45-63 (``--export-quant-cfg`` with int8_sq, fp8, fp8_blockwise, int4_awq,
w4a8_awq, nvfp4 and the two ``*_real_quant`` forms), megatron/core/post_training/modelopt/layers.py:169-249
(``RealQuantTransformerLayer``: weights held in FP8, memory report) and tasks/quantize/calibrate_gpt.py:110-165
(calibration loop).  Here the same recipes are implemented directly:

* every ``ColumnParallelLinear`` / ``RowParallelLinear`` gets an ``input_quantizer`` and a ``weight_quantizer``
  (``TensorQuantizer`` sub-modules, so their ranges travel in the state dict);
* ``quantize(model, fmt, forward_loop)`` runs the loop once in calibration mode (absolute maxima; per input channel
  statistics for the smoothing recipes), reduces the ranges over the tensor-parallel group, folds SmoothQuant / AWQ
  channel scales into the weights, and switches the quantisers to simulated quantisation (quantise-dequantise with a
  straight-through gradient, so quantisation-aware fine-tuning works too);
* ``compress(model)`` replaces the 16-bit weight of every quantised linear by its FP8 image plus scales (per tensor or
  per 128 x 128 block) and reports the bytes saved; on a GPU a per-tensor FP8 weight goes to the FP8 tensor-core
  GEMM as stored (``prequantized_linear``), otherwise the forward de-quantises on the fly;
* ``quantizer_state`` / ``restore_quantizer_state`` describe the attached quantisers so a checkpoint can be loaded
  into a freshly built model.
"""
from __future__ import annotations

import fnmatch
from dataclasses import asdict, dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

FP8_MAX = 448.0
_E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_MID = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


@dataclass
class QuantizerSpec:
    """kind: fp8 | int8 | int4 | nvfp4.  block = (rows, cols) of one scale (cols only for activations);
    axis = 0 gives one scale per output channel; dynamic = ranges taken from the tensor at every call."""
    kind: str = "fp8"
    block: Optional[Tuple[int, int]] = None
    axis: Optional[int] = None
    dynamic: bool = False
    enabled: bool = True


def _spec(kind, **kw):
    return QuantizerSpec(kind=kind, **kw)


# recipe name -> (input quantiser, weight quantiser, smoothing algorithm)
FORMATS: Dict[str, Tuple[QuantizerSpec, QuantizerSpec, Optional[str]]] = {
    "fp8": (_spec("fp8"), _spec("fp8"), None),
    "fp8_blockwise": (_spec("fp8", block=(1, 128), dynamic=True), _spec("fp8", block=(128, 128), dynamic=True), None),
    "fp8_blockwise_32": (_spec("fp8", block=(1, 32), dynamic=True), _spec("fp8", block=(1, 32), dynamic=True), None),
    "int8_sq": (_spec("int8"), _spec("int8", axis=0), "smoothquant"),
    "int4_awq": (_spec("fp8", enabled=False), _spec("int4", block=(1, 128), dynamic=True), "awq_lite"),
    "w4a8_awq": (_spec("fp8"), _spec("int4", block=(1, 128), dynamic=True), "awq_lite"),
    "nvfp4": (_spec("nvfp4", block=(1, 16)), _spec("nvfp4", block=(1, 16)), None),
}
REAL_QUANT = {"fp8_real_quant": "fp8", "fp8_blockwise_real_quant": "fp8_blockwise"}


# ------------------------------------------------------------------------------------------------ number formats
def _e2m1_round(x: torch.Tensor) -> torch.Tensor:
    mid = torch.tensor(_E2M1_MID, dtype=x.dtype, device=x.device)
    grid = torch.tensor(_E2M1_GRID, dtype=x.dtype, device=x.device)
    return grid[torch.bucketize(x.abs().clamp(max=6.0), mid)] * x.sign()


def _qdq(x: torch.Tensor, amax: torch.Tensor, kind: str) -> torch.Tensor:
    """Quantise-dequantise fp32 ``x`` with range ``amax`` (broadcastable)."""
    amax = amax.clamp(min=1e-12)
    if kind == "fp8":
        s = FP8_MAX / amax
        return (x * s).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).to(x.dtype) / s
    if kind == "int8":
        s = 127.0 / amax
        return (x * s).round().clamp(-127, 127) / s
    if kind == "int4":
        s = 7.0 / amax
        return (x * s).round().clamp(-8, 7) / s
    raise ValueError(kind)


def _blocked(x2: torch.Tensor, br: int, bc: int):
    """View a 2-D tensor as [R/br, br, C/bc, bc] after zero padding; returns (view, R, C)."""
    R, C = x2.shape
    pr, pc = (-R) % br, (-C) % bc
    if pr or pc:
        x2 = torch.nn.functional.pad(x2, (0, pc, 0, pr))
    return x2.view((R + pr) // br, br, (C + pc) // bc, bc), R, C


def fake_quant(x: torch.Tensor, spec: QuantizerSpec, amax: Optional[torch.Tensor]) -> torch.Tensor:
    """Values of ``x`` after a round trip through the format of ``spec`` (no gradient logic here)."""
    shape, dtype = x.shape, x.dtype
    x2 = x.reshape(-1, shape[-1]).float()
    if spec.kind == "nvfp4":
        # two levels: a per-tensor fp32 scale (calibrated) and an E4M3 scale per 16 values
        g = (amax.float() if amax is not None else x2.abs().amax()).clamp(min=1e-12) / (6.0 * FP8_MAX)
        v, R, C = _blocked(x2, 1, spec.block[1] if spec.block else 16)
        bmax = v.abs().amax(dim=(1, 3), keepdim=True)
        sb = ((bmax / 6.0 / g).clamp(max=FP8_MAX).to(torch.float8_e4m3fn).float() * g).clamp(min=1e-30)
        out = (_e2m1_round(v / sb) * sb).reshape(v.shape[0] * v.shape[1], -1)[:R, :C]
        return out.reshape(shape).to(dtype)
    if spec.block is not None:
        br, bc = spec.block
        v, R, C = _blocked(x2, br, bc)
        out = _qdq(v, v.abs().amax(dim=(1, 3), keepdim=True), spec.kind)
        return out.reshape(v.shape[0] * v.shape[1], -1)[:R, :C].reshape(shape).to(dtype)
    if spec.axis == 0:
        a = amax.float().view(-1, 1) if amax is not None and not spec.dynamic else x2.abs().amax(dim=1, keepdim=True)
        return _qdq(x2, a, spec.kind).reshape(shape).to(dtype)
    a = amax.float() if amax is not None and not spec.dynamic else x2.abs().amax()
    return _qdq(x2, a, spec.kind).reshape(shape).to(dtype)


# ------------------------------------------------------------------------------------------------ quantiser module
class TensorQuantizer(nn.Module):
    """One quantiser.  States: calibrating (records ranges, passes values through), quantising (simulated
    quantisation with a straight-through gradient) or disabled."""

    def __init__(self, spec: QuantizerSpec, channels: Optional[int] = None):
        super().__init__()
        self.spec = spec
        self.calibrating = False
        self.collect_channels = False
        self.channel_max: Optional[torch.Tensor] = None      # |x| max per input channel (smoothing recipes)
        self.channel_mean: Optional[torch.Tensor] = None
        self._tokens = 0
        self.sample: Optional[torch.Tensor] = None           # a few calibration rows for the AWQ search
        self.register_buffer("_amax", None)
        self.register_buffer("_pre_quant_scale", None)
        self._channels = channels

    # -- buffers that exist only after calibration must also exist before a state dict is loaded
    def materialize(self, amax_shape: Optional[List[int]], pre_quant_channels: Optional[int], device=None):
        if amax_shape is not None:
            self._amax = torch.zeros(amax_shape, dtype=torch.float32, device=device)
        if pre_quant_channels:
            self._pre_quant_scale = torch.ones(pre_quant_channels, dtype=torch.float32, device=device)

    @property
    def amax(self):
        return self._amax

    def _observe(self, x: torch.Tensor):
        x2 = x.detach().reshape(-1, x.shape[-1]).float()
        if self.spec.axis == 0:
            cur = x2.abs().amax(dim=1)
        else:
            cur = x2.abs().amax()
        self._amax = cur if self._amax is None else torch.maximum(self._amax, cur)
        if self.collect_channels:
            cm = x2.abs().amax(dim=0)
            self.channel_max = cm if self.channel_max is None else torch.maximum(self.channel_max, cm)
            sm = x2.abs().sum(dim=0)
            self.channel_mean = sm if self.channel_mean is None else self.channel_mean + sm
            self._tokens += x2.shape[0]
            if self.sample is None:
                self.sample = x2[:512].clone()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._pre_quant_scale is not None:
            x = x * self._pre_quant_scale.to(x.dtype)
        if self.calibrating:
            self._observe(x)
            return x
        if not self.spec.enabled:
            return x
        needs_range = not self.spec.dynamic and (self.spec.block is None or self.spec.kind == "nvfp4")
        if needs_range and self._amax is None:
            return x                                         # never calibrated: leave the tensor alone
        q = fake_quant(x.detach(), self.spec, self._amax)
        return x + (q - x.detach())                          # straight-through estimator

    def extra_repr(self):
        return f"{self.spec.kind} block={self.spec.block} axis={self.spec.axis} enabled={self.spec.enabled}"


class PrequantizedWeight:
    """A compressed weight handed to the FP8 GEMM as it is stored (E4M3 bytes + one fp32 scale)."""
    prequantized = True

    def __init__(self, q: torch.Tensor, scale: torch.Tensor):
        self.q, self.scale, self.shape = q.view(torch.uint8), scale.reshape(1), q.shape


FAST_PATH_CALLS = [0]          # how many linears took the stored-FP8 GEMM (tests read it)


def apply_quantizers(linear, x: torch.Tensor, w: Optional[torch.Tensor]):
    """Called by the tensor-parallel linears when ``linear.ptq`` is set: returns the (x, w) the GEMM sees."""
    if w is None:
        # compressed weight.  On a GPU, without gradients, a per-tensor FP8 weight feeds the FP8 tensor-core GEMM
        # directly (the activation is cast with its own range); otherwise the 16-bit weight is rebuilt on the fly.
        q = linear.weight_q
        if q.is_cuda and linear.weight_scale.numel() == 1 and not torch.is_grad_enabled() \
                and x.dtype in (torch.bfloat16, torch.float16) and not getattr(linear, "ptq_dequantize_only", False) \
                and (x.numel() // x.shape[-1]) % 16 == 0 and q.shape[0] % 16 == 0 and q.shape[1] % 16 == 0:
            FAST_PATH_CALLS[0] += 1
            return x, PrequantizedWeight(q, linear.weight_scale)
        w = dequantize_weight(linear)
    else:
        w = linear.weight_quantizer(w)
    return linear.input_quantizer(x), w


def prequantized_linear(x: torch.Tensor, w: PrequantizedWeight, bias=None, _fmt=None) -> torch.Tensor:
    """y = x W^T with W already in FP8: one cast of the activation, one FP8 GEMM."""
    from ..ops.fp8 import gemm_fp8, quantize
    x2 = x.reshape(-1, x.shape[-1])
    xq = quantize(x2, 0, transpose=False)
    y = gemm_fp8(xq.data, 0, xq.scale_inv, w.q, 0, w.scale, out_dtype=x.dtype,
                 bias=None if bias is None else bias.to(x.dtype))
    return y.view(*x.shape[:-1], w.shape[0])


def quantized_linears(model) -> Iterable[Tuple[str, nn.Module]]:
    from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
    for name, m in model.named_modules():
        if isinstance(m, (ColumnParallelLinear, RowParallelLinear)) and (m.weight is not None or getattr(m, "ptq", False)):
            yield name, m


DEFAULT_SKIP = ("*output_layer*", "*router*", "*lm_head*")


def attach_quantizers(model, fmt: str, skip: Iterable[str] = DEFAULT_SKIP) -> List[str]:
    if fmt not in FORMATS:
        raise ValueError(f"unknown quantisation recipe {fmt!r}; choose from {sorted(FORMATS)}")
    ispec, wspec, _ = FORMATS[fmt]
    done = []
    for name, lin in quantized_linears(model):
        if any(fnmatch.fnmatch(name, p) for p in skip):
            continue
        lin.input_quantizer = TensorQuantizer(QuantizerSpec(**asdict(ispec)))
        lin.weight_quantizer = TensorQuantizer(QuantizerSpec(**asdict(wspec)))
        lin.ptq = True
        lin.ptq_format = fmt
        lin.fp8_eligible = False          # the simulated format decides the numerics, not the FP8 training path
        done.append(name)
    return done


def _tp_max(t: torch.Tensor, group) -> torch.Tensor:
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t


def _awq_search(lin, act_scale: torch.Tensor, grid: int = 11) -> torch.Tensor:
    """AWQ-lite: channel scale s = act_scale^a (normalised); a chosen on a grid to minimise the output error of the
    quantised product on the kept calibration rows."""
    w = lin.weight.detach().float()
    x = lin.input_quantizer.sample
    if x is None:
        return torch.ones_like(act_scale)
    ref = x @ w.t()
    best, best_s = None, torch.ones_like(act_scale)
    for i in range(grid):
        a = i / (grid - 1)
        s = act_scale.clamp(min=1e-8).pow(a)
        s = s / (s.max() * s.min()).sqrt().clamp(min=1e-8)
        wq = fake_quant(w * s, lin.weight_quantizer.spec, None)
        err = ((x / s) @ wq.t() - ref).pow(2).mean().item()
        if best is None or err < best:
            best, best_s = err, s
    return best_s


@torch.no_grad()
def _finish_calibration(model, names: List[str], algo: Optional[str], alpha: float = 0.5):
    from ..parallel.layers import ColumnParallelLinear
    mods = dict(model.named_modules())
    for name in names:
        lin = mods[name]
        iq, wq = lin.input_quantizer, lin.weight_quantizer
        col = isinstance(lin, ColumnParallelLinear)
        group = lin.tp_group if lin.tp_size > 1 else None
        if algo is not None and iq.channel_max is not None:
            if algo == "smoothquant":
                act = _tp_max(iq.channel_max.clone(), group if col else None)
                wmax = _tp_max(lin.weight.detach().float().abs().amax(dim=0), group if col else None)
                s = (act.clamp(min=1e-5).pow(alpha) / wmax.clamp(min=1e-5).pow(1 - alpha)).clamp(min=1e-4, max=1e4)
            else:
                mean = iq.channel_mean / max(iq._tokens, 1)
                if col and group is not None:
                    dist.all_reduce(mean, group=group)
                    mean /= dist.get_world_size(group)
                s = _awq_search(lin, mean)
                if col and group is not None:               # the shards share their input: agree on one scale
                    dist.all_reduce(s, group=group)
                    s /= dist.get_world_size(group)
            lin.weight.data.mul_(s.to(lin.weight.dtype))
            iq._pre_quant_scale = (1.0 / s).float()
            if iq._amax is not None and iq.channel_max is not None and iq.spec.axis is None:
                iq._amax = (iq.channel_max / s).amax()
        # ranges of one logical tensor must agree on every shard of it
        if iq._amax is not None:
            _tp_max(iq._amax, group)
        wq.calibrating = True
        wq(lin.weight)                                       # weight range (after folding)
        if wq._amax is not None and wq.spec.axis is None:
            _tp_max(wq._amax, group)
        for q in (iq, wq):
            q.calibrating = q.collect_channels = False
            q.sample = q.channel_max = q.channel_mean = None


def quantize(model, fmt: str, forward_loop: Optional[Callable] = None, skip: Iterable[str] = DEFAULT_SKIP,
             alpha: float = 0.5) -> List[str]:
    """Attach quantisers of recipe ``fmt``, calibrate them by running ``forward_loop(model)`` and switch to simulated
    quantisation.  Returns the names of the quantised linears."""
    real = fmt in REAL_QUANT
    base = REAL_QUANT.get(fmt, fmt)
    names = attach_quantizers(model, base, skip)
    algo = FORMATS[base][2]
    mods = dict(model.named_modules())
    for n in names:
        mods[n].input_quantizer.calibrating = True
        mods[n].input_quantizer.collect_channels = algo is not None
    if forward_loop is not None:
        was_training = model.training
        model.eval()
        with torch.no_grad():
            forward_loop(model)
        model.train(was_training)
    _finish_calibration(model, names, algo, alpha)
    if real:
        compress(model)
    return names


# ------------------------------------------------------------------------------------------------ real quantisation
@torch.no_grad()
def compress(model) -> Dict[str, int]:
    """Hold the weight of every quantised FP8 linear as FP8 values + fp32 scales instead of 16 bits
    (per tensor, or per 128 x 128 block for the block-wise recipe).  Returns {"before": bytes, "after": bytes}."""
    before = after = 0
    for _, lin in quantized_linears(model):
        if not getattr(lin, "ptq", False) or lin.weight is None or lin.weight_quantizer.spec.kind != "fp8":
            continue
        w = lin.weight.detach()
        before += w.numel() * w.element_size()
        spec = lin.weight_quantizer.spec
        w2 = w.float()
        if spec.block is not None:
            v, R, C = _blocked(w2, *spec.block)
            scale = (v.abs().amax(dim=(1, 3), keepdim=True).clamp(min=1e-12) / FP8_MAX)
            q = (v / scale).clamp(-FP8_MAX, FP8_MAX).reshape(v.shape[0] * v.shape[1], -1)[:R, :C]
            scale = scale.reshape(v.shape[0], v.shape[2])
        else:
            amax = lin.weight_quantizer._amax if lin.weight_quantizer._amax is not None else w2.abs().amax()
            scale = (amax.float().clamp(min=1e-12) / FP8_MAX).reshape(1, 1)
            q = (w2 / scale).clamp(-FP8_MAX, FP8_MAX)
        lin.register_buffer("weight_q", q.to(torch.float8_e4m3fn).contiguous())
        lin.register_buffer("weight_scale", scale.contiguous())
        lin.ptq_weight_dtype = w.dtype
        lin.weight = None
        after += lin.weight_q.numel() + lin.weight_scale.numel() * 4
    return {"before": before, "after": after}


def dequantize_weight(lin) -> torch.Tensor:
    q, scale = lin.weight_q.float(), lin.weight_scale
    spec = lin.weight_quantizer.spec
    if spec.block is not None and scale.numel() > 1:
        br, bc = spec.block
        scale = scale.repeat_interleave(br, 0)[:q.shape[0]].repeat_interleave(bc, 1)[:, :q.shape[1]]
    return (q * scale).to(getattr(lin, "ptq_weight_dtype", torch.bfloat16))


# ------------------------------------------------------------------------------------------------ state
def quantizer_state(model) -> Dict:
    """JSON-serialisable description of the attached quantisers (structure only; values are in the state dict)."""
    mods = {}
    for name, lin in quantized_linears(model):
        if not getattr(lin, "ptq", False):
            continue
        ent = {"format": lin.ptq_format, "real": lin.weight is None}
        for which in ("input", "weight"):
            q = getattr(lin, f"{which}_quantizer")
            ent[which] = {"amax_shape": None if q._amax is None else list(q._amax.shape),
                          "pre_quant_channels": None if q._pre_quant_scale is None else q._pre_quant_scale.numel()}
        if lin.weight is None:
            ent["weight_q_shape"] = list(lin.weight_q.shape)
            ent["weight_scale_shape"] = list(lin.weight_scale.shape)
            ent["weight_dtype"] = str(lin.ptq_weight_dtype).replace("torch.", "")
        mods[name] = ent
    return {"version": 1, "modules": mods}


def restore_quantizer_state(model, state: Dict) -> None:
    """Re-create the quantisers (with buffers of the recorded shapes) on a freshly built model, so that a state dict
    saved from a quantised model loads into it."""
    mods = dict(model.named_modules())
    for name, ent in state.get("modules", {}).items():
        lin = mods[name]
        ispec, wspec, _ = FORMATS[ent["format"]]
        lin.input_quantizer = TensorQuantizer(QuantizerSpec(**asdict(ispec)))
        lin.weight_quantizer = TensorQuantizer(QuantizerSpec(**asdict(wspec)))
        dev = lin.weight.device if lin.weight is not None else None
        for which in ("input", "weight"):
            getattr(lin, f"{which}_quantizer").materialize(ent[which]["amax_shape"], ent[which]["pre_quant_channels"], dev)
        lin.ptq, lin.ptq_format, lin.fp8_eligible = True, ent["format"], False
        if ent.get("real"):
            lin.ptq_weight_dtype = getattr(torch, ent["weight_dtype"])
            lin.register_buffer("weight_q", torch.zeros(ent["weight_q_shape"], device=dev).to(torch.float8_e4m3fn))
            lin.register_buffer("weight_scale", torch.ones(ent["weight_scale_shape"], device=dev))
            lin.weight = None


def disable_quantizers(model) -> None:
    for _, lin in quantized_linears(model):
        if getattr(lin, "ptq", False) and lin.weight is not None:
            lin.ptq = False


def enable_quantizers(model) -> None:
    for _, lin in quantized_linears(model):
        if hasattr(lin, "weight_quantizer"):
            lin.ptq = True
