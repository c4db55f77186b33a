"""Multi-token prediction: extra depth-k heads that predict token t+1+k from the main model's hidden
state and the embedding of token t+k.

Reference: megatron/core/transformer/multi_token_prediction.py (``MultiTokenPredictionLayer`` :391,
``MultiTokenPredictionBlock`` :650, ``roll_tensor`` :106, ``MTPLossAutoScaler`` :262).  Each depth has
two norms (embedding, hidden), a 2h -> h projection, one transformer layer and a final norm; the main
model's embedding and output layer are shared.  The depth losses are averaged, scaled by
``mtp_loss_scaling_factor / mtp_num_layers`` and attached to the main loss so their gradient flows in
the same backward.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..config import TransformerConfig
from ..ops import core as ops
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear
from .moe import save_to_aux_losses_tracker
from .transformer import Norm, TransformerLayer


def roll_tensor(t: torch.Tensor, shifts: int = -1, dim: int = -1):
    """Shift left along ``dim`` and zero the vacated tail; returns (rolled, sum of rolled)."""
    r = torch.roll(t, shifts=shifts, dims=dim)
    idx = [slice(None)] * r.dim()
    idx[dim] = slice(shifts, None) if shifts < 0 else slice(0, shifts)
    r[tuple(idx)] = 0
    return r, r.sum()


class MTPLossAutoScaler(torch.autograd.Function):
    """Identity on the main loss; the MTP loss receives gradient = current loss scale."""
    main_loss_backward_scale: Optional[torch.Tensor] = None

    @staticmethod
    def forward(ctx, output, mtp_loss):
        ctx.save_for_backward(mtp_loss)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (mtp_loss,) = ctx.saved_tensors
        s = MTPLossAutoScaler.main_loss_backward_scale
        if s is None:
            s = torch.ones(1, device=mtp_loss.device)
        return grad_output, torch.ones_like(mtp_loss) * s.to(mtp_loss.device).reshape(()).to(mtp_loss.dtype)

    @staticmethod
    def set_loss_scale(scale: torch.Tensor):
        MTPLossAutoScaler.main_loss_backward_scale = scale


class MultiTokenPredictionLayer(nn.Module):
    def __init__(self, config: TransformerConfig, layer_number: int):
        super().__init__()
        self.config = config
        self.enorm = Norm(config, config.hidden_size)
        self.hnorm = Norm(config, config.hidden_size)
        # the concatenated [embedding ; hidden] is gathered over the sequence first when SP is on
        self.eh_proj = ColumnParallelLinear(2 * config.hidden_size, config.hidden_size, config=config,
                                            init_method=config.init_method, bias=False, gather_output=True)
        self.transformer_layer = TransformerLayer(config, config.num_layers + layer_number)
        self.final_layernorm = Norm(config, config.hidden_size)

    def forward(self, decoder_input, hidden_states, rotary=None):
        x = torch.cat((self.enorm(decoder_input), self.hnorm(hidden_states)), dim=-1)
        x, _ = self.eh_proj(x)
        if self.config.sequence_parallel and state.model_parallel_is_initialized() and \
                state.get_tensor_model_parallel_world_size() > 1:
            from ..parallel.mappings import scatter_to_sequence_parallel_region
            x = scatter_to_sequence_parallel_region(x)
        x = self.transformer_layer(x, rotary=rotary)
        return self.final_layernorm(x)


class MultiTokenPredictionBlock(nn.Module):
    def __init__(self, config: TransformerConfig, vocab_size: int):
        super().__init__()
        self.config, self.vocab_size = config, vocab_size
        self.layers = nn.ModuleList([MultiTokenPredictionLayer(config, i + 1) for i in range(config.mtp_num_layers)])

    def forward(self, hidden_states, input_ids, position_ids, labels, loss_mask, rotary, embedding, output_layer,
                output_weight, loss_fn=None):
        """Returns the scaled sum of the depth losses (a scalar that carries the MTP gradient)."""
        cfg = self.config
        if embedding is None:
            raise RuntimeError("multi-token prediction needs the embedding on the last pipeline stage")
        if loss_mask is None:
            loss_mask = torch.ones_like(labels, dtype=torch.float32)
        total = None
        scale = (cfg.mtp_loss_scaling_factor if cfg.mtp_loss_scaling_factor is not None else 0.1) / cfg.mtp_num_layers
        h = hidden_states
        for depth, layer in enumerate(self.layers):
            input_ids, _ = roll_tensor(input_ids, -1, -1)
            labels, _ = roll_tensor(labels, -1, -1)
            loss_mask, num_tokens = roll_tensor(loss_mask, -1, -1)
            dec_in = embedding(input_ids, position_ids)
            h = layer(dec_in, h, rotary)
            logits, _ = output_layer(h, weight=output_weight)
            per_tok = loss_fn(labels, logits)                                   # [b, s]
            depth_loss = (per_tok * loss_mask).sum() / num_tokens.clamp(min=1)
            if self.training:
                save_to_aux_losses_tracker("mtp_loss", depth_loss / cfg.mtp_num_layers, depth + 1, cfg.mtp_num_layers)
            total = depth_loss * scale if total is None else total + depth_loss * scale
        return total
