"""Layer specs: the reference's spec entry points build this library's layers, per-layer MoE patterns come from
the block spec, and user classes can take a slot.  Mirrors tests/unit_tests/transformer/test_spec_customization.py."""
import copy

import pytest
import torch
import torch.nn as nn

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.gpt import GPTModel
from megatron_lm_b200.models.gpt_layer_specs import (TransformerBlockSubmodules, get_gpt_decoder_block_spec,
                                                     get_gpt_layer_local_spec,
                                                     get_gpt_layer_with_transformer_engine_spec, get_gpt_mtp_block_spec,
                                                     get_mlp_module_spec, layer_spec_is_moe)
from megatron_lm_b200.models.spec_utils import ModuleSpec
from megatron_lm_b200.models.transformer import MLP, IdentityOp, Norm, TransformerLayer


def _cfg(**kw):
    base = dict(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                attention_dropout=0.0, use_cpu_initialization=True, normalization="RMSNorm", gated_linear_unit=True,
                activation_func="silu", add_bias_linear=False)
    base.update(kw)
    return TransformerConfig(**base)


def _run(model):
    ids = torch.arange(24).view(2, 12) % 50
    return model(ids, None, None)


def test_local_spec_builds_the_same_model_as_no_spec():
    cfg = _cfg()
    torch.manual_seed(0)
    a = GPTModel(cfg, 50, 16, position_embedding_type="rope")
    torch.manual_seed(0)
    b = GPTModel(cfg, vocab_size=50, max_sequence_length=16, position_embedding_type="rope",
                 transformer_layer_spec=get_gpt_layer_local_spec())
    torch.manual_seed(0)
    c = GPTModel(cfg, get_gpt_layer_with_transformer_engine_spec(), 50, 16, position_embedding_type="rope")
    assert [n for n, _ in a.named_parameters()] == [n for n, _ in b.named_parameters()] == \
        [n for n, _ in c.named_parameters()]
    out = _run(a)
    assert torch.equal(out, _run(b)) and torch.equal(out, _run(c))
    assert c.vocab_size == 50 and c.max_sequence_length == 16 and c.pre_process


def test_block_spec_places_moe_layers_by_pattern():
    from megatron_lm_b200.models.moe import MoELayer
    cfg = _cfg(num_layers=4, num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=48, moe_layer_freq=[1, 0, 0, 1],
               moe_grouped_gemm=True)
    spec = get_gpt_decoder_block_spec(cfg, use_transformer_engine=True)
    assert isinstance(spec, TransformerBlockSubmodules) and len(spec.layer_specs) == 4
    assert [layer_spec_is_moe(s) for s in spec.layer_specs] == [True, False, False, True]
    m = GPTModel(cfg, 50, 16, position_embedding_type="rope", transformer_layer_spec=spec)
    kinds = [isinstance(l.mlp, MoELayer) for l in m.decoder.layers]
    assert kinds == [True, False, False, True] and [l.is_moe for l in m.decoder.layers] == kinds
    assert _run(m).shape == (2, 12, 50)
    # a spec can also contradict the config's pattern: all layers dense
    dense = GPTModel(cfg, 50, 16, position_embedding_type="rope", transformer_layer_spec=get_gpt_layer_local_spec())
    assert not any(isinstance(l.mlp, MoELayer) for l in dense.decoder.layers)
    with pytest.raises(ValueError):
        GPTModel(cfg, 50, 16, transformer_layer_spec=TransformerBlockSubmodules(layer_specs=spec.layer_specs[:3]))


class _ScaledMLP(nn.Module):
    """A user module for the MLP slot: same call contract (returns output and optional bias)."""

    def __init__(self, config, layer_number, gain: float = 1.0):
        super().__init__()
        self.inner, self.gain, self.layer_number = MLP(config), gain, layer_number

    def forward(self, x):
        y, b = self.inner(x)
        return y * self.gain, b


def test_user_classes_can_take_slots():
    cfg = _cfg()
    spec = copy.deepcopy(get_gpt_layer_local_spec())
    spec.submodules.pre_mlp_layernorm = IdentityOp
    spec.submodules.mlp = ModuleSpec(module=_ScaledMLP, params={"gain": 0.5})
    m = GPTModel(cfg, 50, 16, position_embedding_type="rope", transformer_layer_spec=spec)
    for i, layer in enumerate(m.decoder.layers):
        assert isinstance(layer.pre_mlp_layernorm, IdentityOp) and isinstance(layer.input_layernorm, Norm)
        assert isinstance(layer.mlp, _ScaledMLP) and layer.mlp.gain == 0.5 and layer.mlp.layer_number == i + 1
    assert not any("pre_mlp_layernorm" in n for n, _ in m.named_parameters())
    out = _run(m)
    out.sum().backward()
    assert torch.isfinite(out).all() and m.decoder.layers[0].mlp.inner.linear_fc1.weight.grad is not None

    class MyLayer(TransformerLayer):
        pass
    custom = ModuleSpec(module=MyLayer, submodules=spec.submodules)
    m2 = GPTModel(cfg, 50, 16, position_embedding_type="rope", transformer_layer_spec=custom)
    assert all(type(l) is MyLayer for l in m2.decoder.layers)


def test_mlp_and_mtp_spec_helpers():
    from megatron_lm_b200.models.moe import MoELayer
    assert get_mlp_module_spec().module is MLP
    assert get_mlp_module_spec(num_experts=8, moe_grouped_gemm=True).module is MoELayer
    cfg = _cfg()
    assert get_gpt_mtp_block_spec(cfg, get_gpt_layer_local_spec()) is None
    cfg2 = _cfg(mtp_num_layers=2)
    mtp = get_gpt_mtp_block_spec(cfg2, get_gpt_decoder_block_spec(cfg2))
    assert mtp is not None and len(mtp.submodules) == 2
