"""Retro: retrieval cross-attention is causal at chunk granularity and trains."""
import torch

from megatron_lm_b200.models.retro import RetroConfig, RetroModel, get_retro_decoder_layer_numbers


def test_layer_numbers():
    assert get_retro_decoder_layer_numbers(12) == [6, 9, 12]
    assert get_retro_decoder_layer_numbers(24) == [9, 12, 15, 18, 21, 24]


def test_retro_causality_and_grad():
    torch.manual_seed(0)
    cfg = RetroConfig(num_layers=6, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                      attention_dropout=0.0, retro_chunk_length=4, retro_num_neighbors=2, retro_num_retrieved_chunks=2,
                      retro_encoder_num_layers=1, retro_encoder_hidden_dropout=0.0, retro_encoder_attention_dropout=0.0)
    m = RetroModel(cfg, 64, 32).eval()
    ids = torch.randint(0, 64, (2, 12))
    ctx = torch.randint(0, 64, (2, 3, 2, 8))
    with torch.no_grad():
        a = m(ids, context_input_ids=ctx)
        # neighbours of the last chunk influence nothing before the last token of that chunk
        ctx2 = ctx.clone(); ctx2[:, 2] = 1
        b = m(ids, context_input_ids=ctx2)
        # future tokens do not influence earlier positions
        ids3 = ids.clone(); ids3[:, 8:] = 2
        c = m(ids3, context_input_ids=ctx)
    assert a.shape == (2, 12, 64)
    assert torch.allclose(a[:, :11], b[:, :11], atol=1e-5) and not torch.allclose(a[:, 11], b[:, 11], atol=1e-5)
    assert torch.allclose(a[:, :7], c[:, :7], atol=1e-5)
    m.train()
    m(ids, context_input_ids=ctx, labels=ids).mean().backward()
    p = m.retro_layers["6"].attn.linear_q.weight
    g = p.grad if p.grad is not None else p.main_grad
    assert g.abs().sum() > 0
