import json

import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.heterogeneous import build_heterogeneous_layers
from megatron_lm_b200.models.upcycling import upcycle_state_dict


def test_upcycle_shapes_and_copies():
    sd = {"decoder.layers.0.mlp.linear_fc1.weight": torch.randn(16, 8), "decoder.layers.0.mlp.linear_fc2.weight": torch.randn(8, 8),
          "decoder.layers.0.input_layernorm.weight": torch.ones(8)}
    up = upcycle_state_dict(sd, 4)
    assert up["decoder.layers.0.mlp.experts.weight1"].shape == (4, 16, 8)
    assert torch.equal(up["decoder.layers.0.mlp.experts.weight1"][3], sd["decoder.layers.0.mlp.linear_fc1.weight"])
    assert up["decoder.layers.0.mlp.router.weight"].shape == (4, 8)
    assert "decoder.layers.0.mlp.linear_fc1.weight" not in up
    g = upcycle_state_dict(sd, 4, granularity=2)
    assert g["decoder.layers.0.mlp.experts.weight1"].shape == (4, 8, 8) and g["decoder.layers.0.mlp.experts.weight2"].shape == (4, 8, 4)


def test_heterogeneous_layers():
    cfg = TransformerConfig(num_layers=3, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0)
    blocks = {"block_configs": [
        {"attention": {"n_heads_in_group": 2}, "ffn": {"intermediate_size": 48}},
        {"attention": {"no_op": True}, "ffn": {"replace_with_linear": True}},
        {"attention": {"replace_with_linear": True}, "ffn": {"no_op": True}}]}
    layers = build_heterogeneous_layers(cfg, json.dumps(blocks))
    assert layers[0].self_attention.ng == 2 and layers[0].mlp.linear_fc1.weight.shape[0] == 48
    assert not hasattr(layers[1], "self_attention") and not hasattr(layers[2], "mlp")
    x = torch.randn(6, 2, 32, requires_grad=True)
    h = x
    for l in layers:
        h = l(h)
    h.sum().backward()
    assert h.shape == x.shape and x.grad is not None
