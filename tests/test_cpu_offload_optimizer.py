"""Hybrid host/device optimizer equals one AdamW over all parameters, for any offload fraction."""
import pytest
import torch

from megatron_lm_b200.optimizer.cpu_offload import HybridDeviceOptimizer


@pytest.mark.parametrize("frac", [0.0, 0.4, 1.0])
def test_hybrid_matches_adamw(frac):
    torch.manual_seed(0)
    ws = [torch.randn(n, 8) for n in (4, 16, 6, 10)]
    a = [torch.nn.Parameter(w.clone()) for w in ws]
    b = [torch.nn.Parameter(w.clone()) for w in ws]
    ref = torch.optim.AdamW(a, lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95))
    hyb = HybridDeviceOptimizer(b, offload_fraction=frac, lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95))
    assert (len(hyb.cpu_copy) == 0) == (frac == 0.0)
    for step in range(4):
        for pa, pb in zip(a, b):
            g = torch.randn_like(pa)
            pa.grad = g.clone()
            pb.grad = g.clone()
        if step == 2:
            for g in hyb.param_groups:
                g["lr"] = 5e-3
            for g in ref.param_groups:
                g["lr"] = 5e-3
        ref.step()
        hyb.step()
    for pa, pb in zip(a, b):
        assert torch.allclose(pa, pb, atol=1e-6)
    sd = hyb.state_dict()
    hyb.load_state_dict(sd)
