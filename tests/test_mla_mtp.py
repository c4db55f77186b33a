"""Multi-latent attention and multi-token prediction: shapes, gradients, and the MTP loss definition."""
import torch

from megatron_lm_b200.config import MLATransformerConfig, TransformerConfig
from megatron_lm_b200.models.gpt import GPTModel
from megatron_lm_b200.models.mla import YarnRotaryEmbedding, yarn_get_mscale
from megatron_lm_b200.models.mtp import roll_tensor


def test_roll_tensor():
    t = torch.tensor([[1, 2, 3, 4]])
    r, s = roll_tensor(t, -1, -1)
    assert r.tolist() == [[2, 3, 4, 0]] and int(s) == 9


def test_yarn_tables():
    assert yarn_get_mscale(1.0) == 1.0 and yarn_get_mscale(40.0, 1.0) > 1.0
    plain = YarnRotaryEmbedding(64, scaling_factor=1.0)
    cos, sin = plain(16, "cpu")
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2).float() / 64))
    assert torch.allclose(cos, torch.outer(torch.arange(16.0), inv).cos(), atol=1e-6)
    y = YarnRotaryEmbedding(64, scaling_factor=40.0, original_max_position_embeddings=4096)
    f = y._inv_freq("cpu")
    assert torch.allclose(f[0], inv[0]) and torch.allclose(f[-1], inv[-1] / 40.0)      # fast dims kept, slow dims scaled


def test_mla_model_trains():
    torch.manual_seed(0)
    cfg = MLATransformerConfig(num_layers=2, hidden_size=64, num_attention_heads=4, ffn_hidden_size=128,
                               q_lora_rank=32, kv_lora_rank=24, qk_head_dim=16, qk_pos_emb_head_dim=8, v_head_dim=16,
                               gated_linear_unit=True, add_bias_linear=False, hidden_dropout=0.0, attention_dropout=0.0,
                               rotary_scaling_factor=4.0, original_max_position_embeddings=16)
    m = GPTModel(cfg, vocab_size=64, max_sequence_length=32, position_embedding_type="rope")
    ids = torch.randint(0, 64, (2, 16))
    loss = m(ids, labels=ids).mean()
    loss.backward()
    for n, p in m.named_parameters():
        g = getattr(p, "main_grad", None) if p.grad is None else p.grad
        assert g is not None and torch.isfinite(g).all(), n
    # causality: logits at position t do not depend on later tokens
    m.eval()
    with torch.no_grad():
        a = m(ids)
        ids2 = ids.clone(); ids2[:, 10:] = 1
        b = m(ids2)
    assert torch.allclose(a[:, :10], b[:, :10], atol=1e-5)


def test_mtp_loss_matches_definition():
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            mtp_num_layers=2, mtp_loss_scaling_factor=0.3, hidden_dropout=0.0, attention_dropout=0.0,
                            add_bias_linear=False)
    m = GPTModel(cfg, vocab_size=48, max_sequence_length=16)
    ids = torch.randint(0, 48, (2, 12)); labels = torch.roll(ids, -1, 1)
    mask = torch.ones(2, 12)
    loss = m(ids, labels=labels, loss_mask=mask)
    assert loss.shape == (2, 12)
    loss.mean().backward()
    grads = [p.grad if p.grad is not None else getattr(p, "main_grad", None) for p in m.mtp.parameters()]
    assert all(g is not None and g.abs().sum() > 0 for g in grads)
