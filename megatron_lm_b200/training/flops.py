"""Model FLOPs per iteration, the reference's accounting (megatron/training/training.py:155-436,
dense/MoE formula :354-420): forward+backward = 3 x forward, 2 FLOPs per multiply-add, causal
attention counted at half, logits included, embeddings lookups not."""
from __future__ import annotations


def num_floating_point_operations(*, batch_size: int, seq_length: int, num_layers: int, hidden_size: int,
                                  num_attention_heads: int, num_query_groups=None, kv_channels=None,
                                  ffn_hidden_size=None, padded_vocab_size: int, swiglu: bool = False,
                                  num_experts=None, moe_router_topk: int = 1, moe_ffn_hidden_size=None,
                                  moe_layer_freq=1, moe_shared_expert_intermediate_size=None,
                                  mtp_num_layers=None) -> float:
    ng = num_query_groups or num_attention_heads
    kv = kv_channels or hidden_size // num_attention_heads
    ffn = ffn_hidden_size or 4 * hidden_size
    gate = 1.5 if swiglu else 1.0       # (3/2) x two matrices = three matrices
    query_proj = kv * num_attention_heads
    qp_ratio = query_proj / hidden_size
    if num_experts is None:
        n_moe, n_dense = 0, num_layers
    else:
        if isinstance(moe_layer_freq, int):
            pattern = [1 if i % moe_layer_freq == 0 else 0 for i in range(num_layers)]
        else:
            pattern = list(moe_layer_freq)
        n_moe = sum(pattern)
        n_dense = num_layers - n_moe
    moe_ffn = moe_ffn_hidden_size or ffn
    shared = moe_shared_expert_intermediate_size or 0
    mtp = mtp_num_layers or 0
    expansion = 3 * 2 * 2      # fwd+bwd (x3), multiply-add (x2), two matrices per block part (x2)
    attn = (1 + ng / num_attention_heads + seq_length / hidden_size / 2) * qp_ratio
    mlp = (ffn * n_dense + (moe_ffn * moe_router_topk + shared) * n_moe) / num_layers / hidden_size * gate
    total_layers = num_layers + mtp
    per_layer = expansion * batch_size * seq_length * total_layers * hidden_size * hidden_size * (attn + mlp)
    logits = 3 * 2 * batch_size * seq_length * hidden_size * padded_vocab_size * (mtp + 1)
    mtp_extra = 3 * 2 * batch_size * seq_length * hidden_size * hidden_size * 2 * mtp   # eh_proj per MTP layer
    return float(per_layer + logits + mtp_extra)


def flops_from_config(config, batch_size: int, seq_length: int, padded_vocab_size: int) -> float:
    return num_floating_point_operations(
        batch_size=batch_size, seq_length=seq_length, num_layers=config.num_layers, hidden_size=config.hidden_size,
        num_attention_heads=config.num_attention_heads, num_query_groups=config.num_query_groups,
        kv_channels=config.kv_channels, ffn_hidden_size=config.ffn_hidden_size, padded_vocab_size=padded_vocab_size,
        swiglu=config.gated_linear_unit, num_experts=config.num_moe_experts, moe_router_topk=config.moe_router_topk,
        moe_ffn_hidden_size=config.moe_ffn_hidden_size, moe_layer_freq=config.moe_layer_freq,
        moe_shared_expert_intermediate_size=config.moe_shared_expert_intermediate_size,
        mtp_num_layers=config.mtp_num_layers)
