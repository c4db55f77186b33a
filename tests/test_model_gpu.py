"""Whole-model numerics on the GPU against the same model evaluated in fp32 on the CPU."""
import pytest
import torch

from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig
from megatron_lm_b200.models.gpt import GPTModel
from megatron_lm_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / (b.float().norm() + 1e-12)).item()


def _cfg(kind, dtype, device_cpu):
    kw = dict(num_layers=2, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512, hidden_dropout=0.0,
              attention_dropout=0.0, params_dtype=dtype, bf16=dtype == torch.bfloat16, use_cpu_initialization=device_cpu,
              kv_channels=64)
    if kind == "llama":
        kw.update(normalization="RMSNorm", gated_linear_unit=True, activation_func="silu", add_bias_linear=False,
                  num_query_groups=2)
    return TransformerConfig(**kw)


@pytest.mark.parametrize("kind", ["gpt", "llama"])
def test_loss_and_grads_match_cpu_fp32(kind):
    torch.manual_seed(0)
    V, S, B = 512, 256, 2
    pe = "rope" if kind == "llama" else "learned_absolute"
    ref = GPTModel(_cfg(kind, torch.float32, True), V, S, position_embedding_type=pe,
                   share_embeddings_and_output_weights=(kind == "gpt"))
    gpu = GPTModel(_cfg(kind, torch.bfloat16, False), V, S, position_embedding_type=pe,
                   share_embeddings_and_output_weights=(kind == "gpt"))
    with torch.no_grad():
        for (n, p), (_, q) in zip(ref.named_parameters(), gpu.named_parameters()):
            p.copy_(p.to(torch.bfloat16).float())          # both sides start from bf16-representable weights
            q.copy_(p)
    tokens = torch.randint(0, V, (B, S + 1))
    lr = ref(tokens[:, :-1], labels=tokens[:, 1:]).mean()
    lg = gpu(tokens[:, :-1].cuda(), labels=tokens[:, 1:].cuda()).mean()
    assert abs(lr.item() - lg.item()) < 3e-2, (lr.item(), lg.item())
    lr.backward()
    lg.backward()
    torch.cuda.synchronize()
    _lib.check_status()
    worst = 0.0
    for (n, p), (_, q) in zip(ref.named_parameters(), gpu.named_parameters()):
        assert q.grad is not None, n
        r = _rel(q.grad, p.grad)
        worst = max(worst, r)
        assert r < 8e-2, (n, r)
    assert worst > 0


def test_causality_future_tokens_do_not_change_past_logits():
    torch.manual_seed(1)
    V, S = 512, 384
    m = GPTModel(_cfg("llama", torch.bfloat16, False), V, S, position_embedding_type="rope").eval()
    t1 = torch.randint(0, V, (1, S), device="cuda")
    t2 = t1.clone()
    t2[:, 200:] = torch.randint(0, V, (1, S - 200), device="cuda")
    with torch.no_grad():
        a, b = m(t1), m(t2)
    assert torch.equal(a[:, :200], b[:, :200])
    assert not torch.equal(a[:, 200:], b[:, 200:])


def test_train_step_reduces_loss_and_matches_cpu_trajectory():
    from megatron_lm_b200.training.training import setup_model_and_optimizer, train_step
    torch.manual_seed(2)
    V, S, B = 256, 128, 2
    tokens = torch.randint(0, V, (B, S + 1))
    traj = {}
    for dev in ("cpu", "cuda"):
        torch.manual_seed(3)
        cfg = _cfg("llama", torch.float32 if dev == "cpu" else torch.bfloat16, True)
        cfg.use_cpu_initialization = True

        def provider(pre_process=True, post_process=True, vp_stage=None):
            m = GPTModel(cfg, V, S, position_embedding_type="rope")
            return m.cuda() if dev == "cuda" else m
        model, opt, _ = setup_model_and_optimizer(provider, cfg, OptimizerConfig(lr=2e-3, clip_grad=1.0, weight_decay=0.0),
                                                  DistributedDataParallelConfig(grad_reduce_in_fp32=True))
        tk = tokens.to(dev)

        def fwd(it, m):
            out = m(tk[:, :-1], labels=tk[:, 1:])
            return out, (lambda o: (o.float().mean(), {"lm loss": o.float().mean().detach()}))
        losses = []
        for _ in range(6):
            l, *_ = train_step(fwd, None, model, opt, None, cfg, num_microbatches=1, seq_length=S, micro_batch_size=B)
            losses.append(float(l["lm loss"]))
        traj[dev] = losses
    assert traj["cuda"][-1] < traj["cuda"][0]
    for a, b in zip(traj["cpu"], traj["cuda"]):
        assert abs(a - b) < 0.08, (traj["cpu"], traj["cuda"])


def test_packed_sequences_run_on_the_flash_kernel_per_document():
    """Three documents packed in one row on the GPU: no dense mask is built - each document is one causal
    flash-attention call on a slice of the fused QKV activation - and logits and gradients equal those of the
    documents run one by one."""
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.ops import _lib
    from megatron_lm_b200.packed_seq_params import PackedSeqParams
    torch.manual_seed(3)
    cfg = TransformerConfig(num_layers=2, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512, kv_channels=64,
                            hidden_dropout=0.0, attention_dropout=0.0, normalization="RMSNorm", gated_linear_unit=True,
                            activation_func="silu", add_bias_linear=False, bf16=True, params_dtype=torch.bfloat16)
    m = GPTModel(cfg, vocab_size=512, max_sequence_length=512, position_embedding_type="rope").cuda()
    lens = [130, 57, 200]
    docs = [torch.randint(0, 512, (1, n), device="cuda") for n in lens]
    row = torch.cat(docs, dim=1)
    labels = torch.roll(row, -1, dims=1)
    packed = PackedSeqParams.from_lengths(lens)
    loss = m(row, labels=labels, packed_seq_params=packed)
    loss.float().mean().backward()
    g_packed = m.decoder.layers[0].self_attention.linear_qkv.weight.grad.float().clone() \
        if m.decoder.layers[0].self_attention.linear_qkv.weight.grad is not None else None
    with torch.no_grad():
        both = m(row, packed_seq_params=packed)
        o = 0
        for d in docs:
            alone = m(d)
            n = d.shape[1]
            assert _rel(both[:, o:o + n], alone) < 2e-2, _rel(both[:, o:o + n], alone)
            o += n
        plain = m(row)
    assert _rel(plain[:, lens[0]:], both[:, lens[0]:]) > 5e-2          # without boundaries later documents differ
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.isfinite(loss.float()).all() and (g_packed is None or torch.isfinite(g_packed).all())


@pytest.mark.gpu
def test_activation_offloading_on_gpu_matches_plain_run():
    """Saved tensors of the offloaded layers go to pinned host memory and come back for backward: same loss and
    gradients as the run that keeps them on the device."""
    from megatron_lm_b200.config import TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    base = dict(num_layers=3, hidden_size=256, num_attention_heads=4, ffn_hidden_size=512, hidden_dropout=0.0,
                attention_dropout=0.0, normalization="RMSNorm", gated_linear_unit=True, activation_func="silu",
                add_bias_linear=False, params_dtype=torch.bfloat16, bf16=True)
    ids = torch.randint(0, 128, (2, 128), device="cuda")
    outs = []
    for off in (False, True):
        torch.manual_seed(0)
        cfg = TransformerConfig(cpu_offloading=off, cpu_offloading_num_layers=2 if off else 0, **base)
        m = GPTModel(cfg, 128, 128, parallel_output=False, position_embedding_type="rope").cuda().train()
        loss = m(ids, labels=ids).float().mean()
        loss.backward()
        torch.cuda.synchronize()
        outs.append((loss.item(), {n: p.grad.float().clone() for n, p in m.named_parameters() if p.grad is not None}))
    assert outs[0][0] == outs[1][0]
    assert outs[0][1].keys() == outs[1][1].keys()
    for k in outs[0][1]:
        assert torch.equal(outs[0][1][k], outs[1][1][k]), k
