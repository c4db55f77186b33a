"""Layout rules of the data-parallel parameter / gradient buffers (single process): reverse parameter order,
64-element alignment, bucket closing, padding of bucket ends for the distributed optimizer, equal shard ranges,
parameters and main_grad views aliasing the buffers.  Mirrors the reference's
tests/unit_tests/distributed/test_param_and_grad_buffer.py."""
import math

import pytest
import torch
import torch.nn as nn

from megatron_lm_b200.config import DistributedDataParallelConfig
from megatron_lm_b200.parallel.ddp import ParamAndGradBuffer


def _params(shapes):
    return [nn.Parameter(torch.randn(*s)) for s in shapes]


def _buffer(shapes, dp_size=1, dist_opt=False, bucket_size=None, dp_rank=0):
    cfg = DistributedDataParallelConfig(use_distributed_optimizer=dist_opt, grad_reduce_in_fp32=True)
    ps = _params(shapes)
    vals = [p.detach().clone() for p in ps]
    buf = ParamAndGradBuffer(cfg, ps, torch.float32, torch.float32, None, dp_size, dp_rank, bucket_size, 1.0)
    return buf, ps, vals


def test_parameters_alias_the_buffer_in_reverse_order_on_64_element_boundaries():
    shapes = [(10, 7), (33,), (5, 5, 3), (64,)]
    buf, ps, vals = _buffer(shapes)
    starts = []
    for p, v in zip(ps, vals):
        assert torch.equal(p.data, v)                                  # values survive the move into the buffer
        off = (p.data.data_ptr() - buf.param_data.data_ptr()) // 4
        assert off % 64 == 0 and 0 <= off < buf.param_data.numel()
        assert p.main_grad.data_ptr() - buf.grad_data.data_ptr() == off * 4 and p.main_grad.shape == p.shape
        starts.append(off)
    assert starts == sorted(starts, reverse=True)                      # last parameter first (backward order)
    p = ps[1]
    p.main_grad.fill_(2.0)
    off = starts[1]
    assert torch.equal(buf.grad_data[off:off + 33], torch.full((33,), 2.0))
    buf.zero_grads()
    assert float(buf.grad_data.abs().sum()) == 0.0


def test_buckets_close_at_the_size_and_cover_the_buffer():
    shapes = [(100,), (100,), (100,), (100,), (100,)]                  # 128 elements each after alignment
    buf, ps, _ = _buffer(shapes, bucket_size=250)
    assert len(buf.buckets) >= 2
    assert buf.buckets[0].start == 0 and buf.buckets[-1].end == buf.grad_data.numel()
    for a, b in zip(buf.buckets, buf.buckets[1:]):
        assert a.end == b.start
    for b in buf.buckets[:-1]:
        assert b.end - b.start >= 250
    assert sorted(id(p) for b in buf.buckets for p in b.params) == sorted(id(p) for p in ps)
    one, _, _ = _buffer(shapes, bucket_size=None)
    assert len(one.buckets) == 1


@pytest.mark.parametrize("dp", [2, 3, 8])
def test_distributed_optimizer_pads_buckets_to_equal_shards(dp):
    shapes = [(1000,), (77, 3), (513,)]
    buf, _, _ = _buffer(shapes, dp_size=dp, dist_opt=True, bucket_size=1100)
    unit = math.lcm(dp, 128)
    for b in buf.buckets:
        assert (b.end - b.start) % unit == 0
        ranges = [buf.shard_range(b, r) for r in range(dp)]
        assert ranges[0][0] == b.start and ranges[-1][1] == b.end
        sizes = {e - s for s, e in ranges}
        assert len(sizes) == 1
        for (s0, e0), (s1, e1) in zip(ranges, ranges[1:]):
            assert e0 == s1
    plain, _, _ = _buffer(shapes, dp_size=dp, dist_opt=False, bucket_size=1100)
    assert plain.grad_data.numel() <= buf.grad_data.numel()
