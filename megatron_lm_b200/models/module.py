"""Module base classes (reference: megatron/core/transformer/module.py:27-258)."""
from __future__ import annotations

import torch
import torch.nn as nn

from ..parallel import state

_FLOAT = (torch.float32,)
_HALF = (torch.float16, torch.bfloat16)


class MegatronModule(nn.Module):
    def __init__(self, config=None):
        super().__init__()
        self.config = config

    def state_dict_for_save_checkpoint(self, prefix: str = "", keep_vars: bool = False):
        return self.state_dict(prefix=prefix, keep_vars=keep_vars)

    def sharded_state_dict(self, prefix: str = "", sharded_offsets=(), metadata=None):
        from ..checkpoint.sharded import model_sharded_state_dict
        init = state.model_parallel_is_initialized()
        return model_sharded_state_dict(
            self, prefix, tp_rank=state.get_tensor_model_parallel_rank() if init else 0,
            tp_size=state.get_tensor_model_parallel_world_size() if init else 1,
            dp_rank=state.get_data_parallel_rank(with_context_parallel=True) if init else 0,
            pp_layer_offset=getattr(getattr(self, "decoder", None), "layer_offset", 0),
            num_layers_global=getattr(self.config, "num_layers", None))

    def set_is_first_microbatch(self):
        for m in self.modules():
            if hasattr(m, "is_first_microbatch"):
                m.is_first_microbatch = True


def _convert(val, fn):
    if isinstance(val, (tuple, list)):
        out = [_convert(v, fn) for v in val]
        return tuple(out) if isinstance(val, tuple) else out
    return fn(val)


class Float16Module(MegatronModule):
    """Casts a module to fp16/bf16; floating inputs are cast down on the first pipeline stage and
    outputs cast back to fp32 on the last."""

    def __init__(self, config, module: nn.Module):
        super().__init__(config)
        if config.fp16:
            self.dtype = torch.float16
        elif config.bf16:
            self.dtype = torch.bfloat16
        else:
            raise ValueError("Float16Module needs fp16 or bf16")
        self.add_module("module", module.to(self.dtype))

    def set_input_tensor(self, t):
        return self.module.set_input_tensor(t)

    def forward(self, *inputs, **kwargs):
        first = state.is_pipeline_first_stage() if state.model_parallel_is_initialized() else True
        last = state.is_pipeline_last_stage() if state.model_parallel_is_initialized() else True
        down = lambda v: v.to(self.dtype) if torch.is_tensor(v) and v.dtype in _FLOAT else v
        up = lambda v: v.float() if torch.is_tensor(v) and v.dtype in _HALF else v
        if first:
            inputs = _convert(inputs, down)
        out = self.module(*inputs, **kwargs)
        return _convert(out, up) if last else out

    def state_dict(self, *a, **kw):
        return self.module.state_dict(*a, **kw)

    def load_state_dict(self, sd, strict=True):
        return self.module.load_state_dict(sd, strict=strict)
