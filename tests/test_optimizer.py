"""Optimizer stack on CPU: learning-rate / weight-decay schedules, loss-scale dynamics, the flat mixed-precision
AdamW against torch.optim.AdamW, gradient clipping, skipped steps on overflow, state round trip.
Mirrors the reference's tests/unit_tests/test_optimizer*.py and test_optimizer_param_scheduler.py."""
import math

import pytest
import torch

from megatron_lm_b200.optimizer.grad_scaler import ConstantGradScaler, DynamicGradScaler
from megatron_lm_b200.optimizer.scheduler import OptimizerParamScheduler


class _Opt:
    def __init__(self, n=1):
        self.param_groups = [dict(lr=0.0, weight_decay=0.0) for _ in range(n)]


def _sched(**kw):
    base = dict(init_lr=0.0, max_lr=1.0, min_lr=0.1, lr_warmup_steps=10, lr_decay_steps=110, lr_decay_style="cosine",
                start_wd=0.0, end_wd=0.0, wd_incr_steps=100, wd_incr_style="constant")
    base.update(kw)
    opt = _Opt()
    return OptimizerParamScheduler(opt, **base), opt


def test_warmup_is_linear_from_init_lr():
    s, opt = _sched(init_lr=0.2)
    s.step(5)
    assert opt.param_groups[0]["lr"] == pytest.approx(0.2 + 0.8 * 0.5)
    s.step(5)
    assert opt.param_groups[0]["lr"] == pytest.approx(1.0)


@pytest.mark.parametrize("style,mid", [("linear", 0.55), ("cosine", 0.55), ("constant", 1.0)])
def test_decay_styles(style, mid):
    s, opt = _sched(lr_decay_style=style)
    s.step(60)                                            # half way through the decay window
    assert opt.param_groups[0]["lr"] == pytest.approx(mid)
    s.step(50)
    assert opt.param_groups[0]["lr"] == pytest.approx(1.0 if style == "constant" else 0.1)
    s.step(500)
    assert opt.param_groups[0]["lr"] == pytest.approx(1.0 if style == "constant" else 0.1)


def test_inverse_square_root_and_wsd():
    s, opt = _sched(lr_decay_style="inverse-square-root", min_lr=0.0, lr_decay_steps=10000)
    s.step(40)
    assert opt.param_groups[0]["lr"] == pytest.approx(math.sqrt(10) / math.sqrt(40))
    for style, want in (("linear", 0.55), ("cosine", 0.55), ("minus_sqrt", 0.1 + 0.9 * (1 - math.sqrt(0.5))),
                        ("exponential", 0.1 + 0.9 * (2 * 0.5 ** 0.5 - 1))):
        s, opt = _sched(lr_decay_style="WSD", wsd_decay_steps=20, lr_wsd_decay_style=style)
        s.step(80)
        assert opt.param_groups[0]["lr"] == pytest.approx(1.0)          # stable phase
        s.step(20)                                                      # half of the final anneal
        assert opt.param_groups[0]["lr"] == pytest.approx(want)


def test_weight_decay_ramp_and_per_group_lr_bounds():
    s, opt = _sched(start_wd=0.0, end_wd=0.2, wd_incr_style="linear", wd_incr_steps=100)
    opt.param_groups.append(dict(lr=0.0, weight_decay=0.0, max_lr=0.5, min_lr=0.05))
    s.step(50)
    assert opt.param_groups[0]["weight_decay"] == pytest.approx(0.1)
    s2, _ = _sched(start_wd=0.0, end_wd=0.2, wd_incr_style="cosine", wd_incr_steps=100)
    s2.step(50)
    assert s2.get_wd() == pytest.approx(0.1)
    s.step(10)
    assert opt.param_groups[1]["lr"] < opt.param_groups[0]["lr"]        # own max_lr
    s.step(1000)
    assert opt.param_groups[1]["lr"] == pytest.approx(0.05)


def test_scheduler_validation_and_checkpoint_rules():
    with pytest.raises(ValueError):
        _sched(lr_warmup_steps=200)
    with pytest.raises(ValueError):
        _sched(lr_decay_style="WSD")
    with pytest.raises(ValueError):
        _sched(min_lr=2.0)
    s, _ = _sched()
    s.step(30)
    sd = s.state_dict()
    s2, opt2 = _sched(max_lr=0.7)                       # default: checkpoint values win
    s2.load_state_dict(sd)
    assert s2.num_steps == 30 and s2.max_lr == 1.0 and opt2.param_groups[0]["lr"] == pytest.approx(s.get_lr({}))
    s3, _ = _sched(max_lr=0.7, use_checkpoint_opt_param_scheduler=False, override_opt_param_scheduler=True)
    s3.load_state_dict(sd)
    assert s3.max_lr == 0.7 and s3.num_steps == 30      # override: class values win, position is restored
    s4, _ = _sched(max_lr=0.7, use_checkpoint_opt_param_scheduler=False)
    with pytest.raises(ValueError):
        s4.load_state_dict(sd)


def test_dynamic_loss_scale_hysteresis_growth_and_floor():
    g = DynamicGradScaler(initial_scale=1024.0, min_scale=256.0, growth_factor=2.0, backoff_factor=0.5,
                          growth_interval=3, hysteresis=2)
    g.update(True)
    assert g.scale == 1024.0                             # first overflow is tolerated
    g.update(True)
    assert g.scale == 512.0
    g.update(True)
    g.update(True)
    assert g.scale == 256.0                              # never below the floor
    for _ in range(3):
        g.update(False)
    assert g.scale == 512.0
    g.update(False)
    g.update(True)                                       # an overflow resets the clean-step count
    g.update(False)
    g.update(False)
    assert g.scale == 512.0
    sd = g.state_dict()
    h = DynamicGradScaler(2.0, 1.0, 2.0, 0.5, 3, 2)
    h.load_state_dict(sd)
    h.update(False)
    assert h.scale == 1024.0
    with pytest.raises(ValueError):
        DynamicGradScaler(1.0, 2.0, 2.0, 0.5, 3, 2)
    c = ConstantGradScaler(128.0)
    c.update(True)
    assert c.scale == 128.0


# ------------------------------------------------------------------------------------------------ optimizer
def _setup(opt_kw=None, params_dtype=torch.float32, ddp_kw=None):
    from megatron_lm_b200.config import DistributedDataParallelConfig, OptimizerConfig, TransformerConfig
    from megatron_lm_b200.models.gpt import GPTModel
    from megatron_lm_b200.training.training import setup_model_and_optimizer
    torch.manual_seed(0)
    cfg = TransformerConfig(num_layers=2, hidden_size=32, num_attention_heads=4, ffn_hidden_size=64, hidden_dropout=0.0,
                            attention_dropout=0.0, use_cpu_initialization=True, params_dtype=params_dtype,
                            bf16=params_dtype == torch.bfloat16)

    def provider(pre_process=True, post_process=True, vp_stage=None):
        return GPTModel(cfg, 64, 16, pre_process=pre_process, post_process=post_process)
    kw = dict(lr=1e-2, weight_decay=0.1, adam_beta1=0.9, adam_beta2=0.95, adam_eps=1e-8, clip_grad=0.0,
              bf16=params_dtype == torch.bfloat16)
    kw.update(opt_kw or {})
    model, opt, _ = setup_model_and_optimizer(provider, cfg, OptimizerConfig(**kw),
                                              DistributedDataParallelConfig(grad_reduce_in_fp32=True, **(ddp_kw or {})))
    return cfg, model, opt


def _loss(model, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 64, (2, 17), generator=g)
    pos = torch.arange(16).unsqueeze(0).expand(2, 16)
    return model(ids[:, :-1], pos, None, labels=ids[:, 1:]).float().mean()


def _step(model, opt, seed, scale=1.0):
    for m in model:
        m.zero_grad_buffer()
    opt.zero_grad()
    (_loss(model[0], seed) * scale).backward()
    for m in model:
        m.finish_grad_sync()
    return opt.step()


def test_adamw_matches_torch_with_no_decay_groups():
    from megatron_lm_b200.models.gpt import GPTModel
    cfg, model, opt = _setup()
    ref = GPTModel(cfg, 64, 16)
    ref.load_state_dict(model[0].module.state_dict())
    decay = [p for n, p in ref.named_parameters() if not (n.endswith(".bias") or p.dim() == 1)]
    no_decay = [p for n, p in ref.named_parameters() if (n.endswith(".bias") or p.dim() == 1)]
    assert decay and no_decay
    topt = torch.optim.AdamW([dict(params=decay, weight_decay=0.1), dict(params=no_decay, weight_decay=0.0)],
                             lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for seed in range(4):
        ok, norm, _ = _step(model, opt, seed)
        assert ok
        topt.zero_grad()
        _loss(ref, seed).backward()
        tnorm = torch.sqrt(sum(p.grad.float().pow(2).sum() for p in ref.parameters()))
        assert float(norm) == pytest.approx(float(tnorm), rel=1e-4)
        topt.step()
    for (n, p), (_, q) in zip(model[0].module.named_parameters(), ref.named_parameters()):
        if n.endswith("linear_qkv.bias"):
            # the key bias has an exactly-zero gradient in exact arithmetic (softmax is shift invariant), so
            # Adam normalises rounding noise there and the two runs need not agree
            continue
        assert torch.allclose(p, q, atol=5e-6, rtol=1e-5), (n, (p - q).abs().max())


def test_clip_grad_scales_the_update():
    _, m1, o1 = _setup(dict(clip_grad=0.0, weight_decay=0.0, optimizer="sgd", sgd_momentum=0.0, lr=0.1))
    _, m2, o2 = _setup(dict(clip_grad=0.05, weight_decay=0.0, optimizer="sgd", sgd_momentum=0.0, lr=0.1))
    before = [p.detach().clone() for p in m1[0].module.parameters()]
    _, n1, _ = _step(m1, o1, 0)
    _, n2, _ = _step(m2, o2, 0)
    assert float(n1) == pytest.approx(float(n2), rel=1e-6) and float(n1) > 0.05
    ratio = 0.05 / (float(n1) + 1e-6)
    for b, p, q in zip(before, m1[0].module.parameters(), m2[0].module.parameters()):
        assert torch.allclose((q - b), (p - b) * ratio, atol=1e-7, rtol=1e-4)


def test_bf16_params_follow_fp32_master_weights():
    _, model, opt = _setup(params_dtype=torch.bfloat16)
    assert all(p.dtype == torch.bfloat16 for p in model[0].module.parameters())
    for seed in range(3):
        _step(model, opt, seed)
    for st in opt.states:
        assert st.master.dtype == torch.float32
        for (s, e, l0) in st.ranges:
            assert torch.equal(st.buf.param_data[s:e], st.master[l0:l0 + e - s].to(torch.bfloat16))


def test_overflow_skips_the_step_and_backs_off_the_scale():
    _, model, opt = _setup(dict(fp16=True, bf16=False, initial_loss_scale=2.0 ** 10, min_loss_scale=1.0,
                                loss_scale_window=2, hysteresis=1))
    before = [p.detach().clone() for p in model[0].module.parameters()]
    for m in model:
        m.zero_grad_buffer()
    opt.zero_grad()
    opt.scale_loss(_loss(model[0], 0)).backward()
    model[0].buffers[0].grad_data[3] = float("inf")
    for m in model:
        m.finish_grad_sync()
    ok, _, _ = opt.step()
    assert not ok and float(opt.get_loss_scale()) == 2.0 ** 9
    assert all(torch.equal(b, p) for b, p in zip(before, model[0].module.parameters()))
    # clean steps: the update is un-scaled and the scale grows back after the window
    for seed in (1, 2):
        for m in model:
            m.zero_grad_buffer()
        opt.zero_grad()
        opt.scale_loss(_loss(model[0], seed)).backward()
        for m in model:
            m.finish_grad_sync()
        ok, norm, _ = opt.step()
        assert ok and float(norm) < 100.0
    assert float(opt.get_loss_scale()) == 2.0 ** 10
    assert any(not torch.equal(b, p) for b, p in zip(before, model[0].module.parameters()))


def test_optimizer_state_round_trip():
    _, model, opt = _setup()
    for seed in range(2):
        _step(model, opt, seed)
    import copy
    sd = copy.deepcopy(opt.state_dict())          # the state dict references live tensors
    msd = {k: v.clone() for k, v in model[0].module.state_dict().items() if torch.is_tensor(v)}
    _step(model, opt, 7)
    after = [p.detach().clone() for p in model[0].module.parameters()]
    _, model2, opt2 = _setup()
    model2[0].module.load_state_dict(msd, strict=False)
    opt2.load_state_dict(sd)
    _step(model2, opt2, 7)
    for a, p in zip(after, model2[0].module.parameters()):
        assert torch.allclose(a, p, atol=1e-6)
