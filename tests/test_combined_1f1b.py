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
