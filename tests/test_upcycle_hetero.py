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


def _dense_and_moe(granularity=1, grouped=True):
    from megatron_lm_b200.models.gpt import GPTModel
    base = dict(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                attention_dropout=0.0, gated_linear_unit=True, activation_func="silu", add_bias_linear=False,
                normalization="RMSNorm", use_cpu_initialization=True)
    torch.manual_seed(0)
    dense = GPTModel(TransformerConfig(**base), 64, 16, parallel_output=False, share_embeddings_and_output_weights=False)
    moe_cfg = TransformerConfig(**base, num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=64 // granularity,
                                moe_grouped_gemm=grouped, moe_token_dispatcher_type="allgather")
    torch.manual_seed(1)
    moe = GPTModel(moe_cfg, 64, 16, parallel_output=False, share_embeddings_and_output_weights=False)
    return dense, moe


def test_upcycled_model_reproduces_the_dense_model():
    import pytest
    from megatron_lm_b200.models.upcycling import upcycle_model
    ids = torch.randint(0, 64, (2, 16))
    pos = torch.arange(16).unsqueeze(0).expand(2, 16)
    for grouped in (True, False):
        for g in (1, 2):
            dense, moe = _dense_and_moe(g, grouped)
            rep = upcycle_model(dense, moe, granularity=g)
            assert sum(v == "router init" for v in rep.values()) == 2
            assert not [k for k, v in rep.items() if v == "kept"], rep
            with torch.no_grad():
                a, b = dense(ids, pos, None), moe(ids, pos, None)
            if g == 1:
                # identical experts, top-k weights that sum to one: the mixture is the dense MLP
                assert torch.allclose(a, b, atol=1e-5), (grouped, (a - b).abs().max())
            else:
                assert torch.isfinite(b).all() and b.shape == a.shape
    dense, moe = _dense_and_moe(1)
    with pytest.raises(ValueError):
        upcycle_model(dense, moe, granularity=3)


def test_gpt_model_from_a_heterogeneous_block_configuration(tmp_path):
    """The block configuration reaches the model through the transformer config (and the command line): pipeline
    stages take their slice of it, and the model trains."""
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.training import arguments as A
    blocks = {"block_configs": [
        {"attention": {"n_heads_in_group": 2}, "ffn": {"intermediate_size": 48}},
        {"attention": {"no_op": True}, "ffn": {"replace_with_linear": True}},
        {"attention": {"replace_with_linear": True}, "ffn": {"no_op": True}},
        {"attention": {}, "ffn": {"ffn_mult": 1.0}}]}
    path = tmp_path / "blocks.json"
    path.write_text(json.dumps(blocks))
    args = A.parse_args(argv=["--num-layers", "4", "--hidden-size", "32", "--num-attention-heads", "4", "--seq-length", "16",
                              "--micro-batch-size", "1", "--train-iters", "1", "--lr", "1e-3",
                              "--heterogeneous-layers-config-path", str(path), "--use-cpu-initialization",
                              "--attention-dropout", "0", "--hidden-dropout", "0"])
    args.world_size, args.rank = 1, 0
    args = A.validate_args(args)
    cfg = A.core_transformer_config_from_args(args)
    assert json.loads(cfg.heterogeneous_layers_config_encoded_json) == blocks
    m = GPTModel(cfg, 64, 16, parallel_output=False)
    layers = m.decoder.layers
    assert len(layers) == 4 and layers[0].mlp.linear_fc1.weight.shape[0] == 48
    assert not hasattr(layers[1], "self_attention") and not hasattr(layers[2], "mlp")
    assert layers[3].mlp.linear_fc1.weight.shape[0] == 256          # 2/3 * 32 rounded up to a multiple of 256
    ids = torch.randint(0, 64, (2, 16))
    loss = m(ids, labels=ids).mean()
    loss.backward()
    assert torch.isfinite(loss) and layers[2].self_attention.linear.weight.grad is not None
