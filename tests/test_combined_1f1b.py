"""The interleaved forward/backward schedule reproduces the plain no-pipelining schedule (losses and gradients)
for a dense and a mixture-of-experts model."""
import pytest
import torch

from megatron_lm_b200.config import TransformerConfig
from megatron_lm_b200.models.gpt import GPTModel
from megatron_lm_b200.parallel.combined_1f1b import ModelChunkSchedulePlan, combined_1f1b_schedule_for_no_pipelining
from megatron_lm_b200.parallel.schedules import forward_backward_no_pipelining


def _model(moe):
    torch.manual_seed(0)
    kw = dict(num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=32, moe_aux_loss_coeff=0.0,
              moe_token_dispatcher_type="alltoall") if moe else {}
    cfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                            hidden_dropout=0.0, attention_dropout=0.0, add_bias_linear=False, **kw)
    return cfg, GPTModel(cfg, 64, 16)


@pytest.mark.parametrize("moe", [False, True])
def test_combined_equals_plain(moe):
    g = torch.Generator().manual_seed(1)
    data = [torch.randint(0, 64, (2, 13), generator=g) for _ in range(3)]

    def loss_func(out):
        l = out.float().mean()
        return l, {"lm loss": l.detach()}

    def run(combined):
        cfg, m = _model(moe)
        it = iter(data)

        def fwd(iterator, model, return_schedule_plan=False):
            t = next(iterator)
            if return_schedule_plan:
                return ModelChunkSchedulePlan(model, t[:, :-1], None, t[:, 1:]), loss_func
            return model(t[:, :-1], labels=t[:, 1:]), loss_func
        f = combined_1f1b_schedule_for_no_pipelining if combined else forward_backward_no_pipelining
        reports = f(forward_step_func=fwd, data_iterator=it, model=[m], num_microbatches=3, seq_length=12,
                    micro_batch_size=2)
        return [float(r["lm loss"]) for r in reports], {n: p.grad.clone() for n, p in m.named_parameters()}
    la, ga = run(False)
    lb, gb = run(True)
    assert la == pytest.approx(lb, abs=1e-6)
    for n in ga:
        assert torch.allclose(ga[n], gb[n], atol=1e-6), n


@pytest.mark.parametrize("moe", [False, True])
def test_delayed_weight_gradients_give_the_same_result(moe):
    """delay_wgrad_compute: backward queues the linears' weight-gradient products, the schedule runs them after the
    forward node that follows; losses and gradients equal the plain schedule's, the queue ends empty."""
    from megatron_lm_b200.parallel import layers
    with pytest.raises(ValueError):
        TransformerConfig(num_layers=1, hidden_size=32, num_attention_heads=4, delay_wgrad_compute=True)
    g = torch.Generator().manual_seed(1)
    data = [torch.randint(0, 64, (2, 13), generator=g) for _ in range(3)]

    def loss_func(out):
        l = out.float().mean()
        return l, {"lm loss": l.detach()}

    def run(delayed):
        torch.manual_seed(0)
        kw = dict(num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=32, moe_aux_loss_coeff=0.0,
                  moe_token_dispatcher_type="alltoall") if moe else {}
        if delayed:
            kw.update(delay_wgrad_compute=True, overlap_moe_expert_parallel_comm=True)
        cfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64,
                                hidden_dropout=0.0, attention_dropout=0.0, add_bias_linear=False, **kw)
        m = GPTModel(cfg, 64, 16)
        deferred = [n for n, p in m.named_parameters() if getattr(p, "defer_wgrad", False)]
        assert bool(deferred) == delayed and all(".layers." in n for n in deferred)
        it = iter(data)
        seen = []
        real = layers.drain_deferred_wgrads

        def counting(*a, **kw2):
            n = real(*a, **kw2)
            seen.append(n)
            return n
        import megatron_lm_b200.parallel.combined_1f1b as c
        c.drain_deferred_wgrads = counting

        def fwd(iterator, model, return_schedule_plan=False):
            t = next(iterator)
            if return_schedule_plan:
                return ModelChunkSchedulePlan(model, t[:, :-1], None, t[:, 1:]), loss_func
            return model(t[:, :-1], labels=t[:, 1:]), loss_func
        try:
            f = combined_1f1b_schedule_for_no_pipelining if delayed else forward_backward_no_pipelining
            reports = f(forward_step_func=fwd, data_iterator=it, model=[m], num_microbatches=3, seq_length=12,
                        micro_batch_size=2)
        finally:
            c.drain_deferred_wgrads = real
        assert not layers._DEFERRED_WGRADS
        if delayed:
            assert sum(seen) == 3 * len(deferred)               # every queued product ran, once per micro-batch
            assert m.decoder.layers[0].backward_dw() == 0
        return [float(r["lm loss"]) for r in reports], {n: p.grad.clone() for n, p in m.named_parameters()}
    la, ga = run(False)
    lb, gb = run(True)
    assert la == pytest.approx(lb, abs=1e-6)
    for n in ga:
        assert torch.allclose(ga[n], gb[n], atol=1e-6), n
