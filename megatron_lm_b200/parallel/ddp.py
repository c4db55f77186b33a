"""Data-parallel wrapper over contiguous parameter / gradient buffers.

Layout rules follow the reference so that shard ranges, checkpoints and
performance characteristics are comparable
(megatron/core/distributed/param_and_grad_buffer.py:489-855,
distributed_data_parallel.py:43-419): one buffer per (param dtype, grad dtype,
expert?) set; parameters are placed in reverse ``module.parameters()`` order
(roughly backward order); each parameter starts on a 64-element boundary; a
bucket closes once it holds at least ``bucket_size`` elements; with the
distributed optimizer every bucket end is padded to a multiple of lcm(dp, 128)
so that each data-parallel rank owns an equal, contiguous 1/dp slice.

Differences by design: parameters signal readiness explicitly (the ops write
``main_grad`` themselves and call ``param.grad_ready``), so there are no autograd
accumulator hooks for them; a fallback hook covers parameters whose gradient is
produced by plain autograd.  Model weights live in one contiguous buffer too,
which lets the optimizer update and re-gather them with single launches.
"""
from __future__ import annotations

import math
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import state
from ..config import DistributedDataParallelConfig, TransformerConfig
from ..ops.optim import scale_


def _pad(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclass
class Bucket:
    index: int
    start: int                      # offset in the buffer (elements)
    end: int                        # exclusive, includes padding
    params: List[nn.Parameter] = field(default_factory=list)


def _single_node() -> bool:
    """Peer memory only reaches GPUs of this node: true when the launcher says every rank of the job is local."""
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    return local >= world


class ParamAndGradBuffer:
    """One contiguous parameter buffer and one gradient buffer, partitioned into buckets."""

    def __init__(self, ddp_config: DistributedDataParallelConfig, params: List[nn.Parameter], param_dtype,
                 grad_dtype, dp_group, dp_size: int, dp_rank: int, bucket_size: Optional[int],
                 gradient_scaling_factor: float, is_expert: bool = False, inter_group=None):
        self.ddp_config, self.param_dtype, self.grad_dtype = ddp_config, param_dtype, grad_dtype
        self.dp_group, self.dp_size, self.dp_rank = dp_group, dp_size, dp_rank
        self.gradient_scaling_factor = gradient_scaling_factor
        self.is_expert = is_expert
        # several distributed-optimizer instances: dp_group is one instance (shards live inside it); the reduced
        # shards are then summed across instances over inter_group
        self.inter_group = inter_group
        self.use_dist_opt = ddp_config.use_distributed_optimizer
        pad_to = 1
        if self.use_dist_opt:
            pad_to = math.lcm(dp_size, 128)
            if ddp_config.pad_buckets_for_high_nccl_busbw:
                pad_to = math.lcm(pad_to, 2 ** 16)
        self.param_index_map: Dict[nn.Parameter, Tuple[int, int, int]] = {}
        self.buckets: List[Bucket] = []
        off = 0
        cur = Bucket(0, 0, 0)

        def close(end_unpadded: int) -> int:
            nonlocal cur
            end = _pad(end_unpadded, pad_to)
            cur.end = end
            self.buckets.append(cur)
            cur = Bucket(len(self.buckets), end, end)
            return end

        for p in reversed(params):
            start = _pad(off, 64)
            # a parameter shared between embedding and output layer gets a bucket of its own
            if getattr(p, "shared_embedding", False) and cur.params:
                off = close(off)
                start = _pad(off, 64)
            end = start + p.numel()
            self.param_index_map[p] = (start, end, cur.index)
            cur.params.append(p)
            off = end
            if (bucket_size is not None and (off - cur.start) >= bucket_size) or getattr(p, "shared_embedding", False):
                off = close(off)
        if cur.params:
            off = close(off)
        self.numel = off
        dev = params[0].device
        # Peer-memory collectives: both buffers live in one symmetric allocation that every rank of the data-
        # parallel group can address, so the gradient reduce-scatter becomes a pull kernel and the optimizer
        # stores updated weights straight into the peers' parameter buffers.
        self.peer = None
        want_peer = getattr(ddp_config, "peer_memory_collectives", False) and self.use_dist_opt and dp_size > 1 \
            and dp_size <= 8 and dev.type == "cuda" and grad_dtype == torch.float32 and param_dtype == torch.bfloat16 \
            and _single_node()
        if want_peer:
            import os
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem
            gbytes = self.numel * 4
            pbytes = _pad(self.numel * 2, 16)
            # one readiness word per (bucket, source rank): rank q stores the step number into word [b][q] of every
            # peer once its bucket b holds this step's complete gradients
            fbytes = _pad(len(self.buckets) * dp_size * 4, 16)
            raw = symm_mem.empty(gbytes + pbytes + fbytes, dtype=torch.uint8, device=dev)
            raw.zero_()
            torch.cuda.synchronize()
            hdl = symm_mem.rendezvous(raw, dp_group)
            base = [int(x) for x in hdl.buffer_ptrs]
            self.grad_data = raw[:gbytes].view(torch.float32)
            self.param_data = raw[gbytes:gbytes + self.numel * 2].view(torch.bfloat16)
            self.peer = {"raw": raw, "hdl": hdl, "grad": base, "param": [b + gbytes for b in base], "pulled": False,
                         "flags": raw[gbytes + pbytes:gbytes + pbytes + len(self.buckets) * dp_size * 4].view(torch.int32),
                         "flag_addr": [b + gbytes + pbytes for b in base], "step": 0, "side": torch.cuda.Stream(),
                         "pending": False}
        else:
            self.param_data = torch.zeros(self.numel, dtype=param_dtype, device=dev)
            self.grad_data = torch.zeros(self.numel, dtype=grad_dtype, device=dev)
        self.params = list(params)
        for p in params:
            s, e, _ = self.param_index_map[p]
            new = self.param_data[s:e].view(p.shape)
            new.copy_(p.data)
            p.data = new
            p.main_grad = self.grad_data[s:e].view(p.shape)
        self.bucket_of = {p: self.buckets[b] for p, (_, _, b) in self.param_index_map.items()}

    # -- shard helpers (distributed optimizer) --------------------------------
    def shard_range(self, bucket: Bucket, rank: Optional[int] = None) -> Tuple[int, int]:
        r = self.dp_rank if rank is None else rank
        n = (bucket.end - bucket.start) // self.dp_size
        return bucket.start + r * n, bucket.start + (r + 1) * n

    def zero_grads(self):
        if self.peer is not None:
            self.peer["hdl"].barrier()          # peers may still be pulling last step's gradients from this buffer
            self.peer["pulled"] = False
        self.grad_data.zero_()

    def peer_barrier(self):
        if self.peer is not None:
            self.peer["hdl"].barrier()


class BucketGroup:
    """Readiness tracking and collectives of one bucket (reference: _ParamAndGradBucketGroup)."""

    def __init__(self, buf: ParamAndGradBuffer, bucket: Bucket):
        self.buf, self.bucket = buf, bucket
        self.ready = set()
        self.counts = {}
        self.grad_handle = None
        self.param_handle = None
        # True from the optimizer step until this bucket's updated shards have been gathered
        self.params_stale = False
        self.pull_count = 0
        self.is_last_microbatch = True
        self.next_group: Optional["BucketGroup"] = None

    def reset(self):
        self.ready.clear()
        self.counts.clear()
        self.grad_handle = None
        self.is_last_microbatch = True

    def register_grad_ready(self, p):
        if not self.is_last_microbatch:
            return
        # a parameter used at several places (tied embedding / output weight on one stage, modules shared with
        # the multi-token-prediction heads) delivers several partial gradients per microbatch, and how many
        # signals that makes depends on which uses run custom kernels and which plain autograd.  Its bucket is
        # therefore not released early: finish_grad_sync reduces it once the backward pass is over.
        if getattr(p, "expected_grad_signals", 1) > 1:
            self.counts[p] = self.counts.get(p, 0) + 1
            return
        if p in self.ready:
            raise RuntimeError("gradient of a parameter signalled ready twice in one microbatch")
        self.ready.add(p)
        if len(self.ready) == len(self.bucket.params) and self.buf.ddp_config.overlap_grad_reduce:
            self.start_grad_sync()

    def start_grad_sync(self):
        if self.grad_handle is not None:
            return
        buf, b = self.buf, self.bucket
        g = buf.grad_data[b.start:b.end]
        if buf.ddp_config.check_for_nan_in_grad:
            if not torch.isfinite(g.float().sum()):
                raise RuntimeError(f"non-finite gradient in bucket {b.index} before the data-parallel reduction")
        if buf.peer is not None:
            self._peer_pull()
            self.grad_handle = "peer"
            return
        if buf.gradient_scaling_factor != 1.0:
            scale_(g, buf.gradient_scaling_factor)
        if buf.dp_size == 1 or buf.dp_group is None:
            self.grad_handle = True
            return
        op = dist.ReduceOp.AVG if buf.ddp_config.average_in_collective else dist.ReduceOp.SUM
        async_op = buf.ddp_config.overlap_grad_reduce
        if buf.use_dist_opt:
            s, e = buf.shard_range(b)
            h = dist.reduce_scatter_tensor(buf.grad_data[s:e], g, op=op, group=buf.dp_group, async_op=async_op)
            self.inter_pending = buf.inter_group is not None
        else:
            h = dist.all_reduce(g, op=op, group=buf.dp_group, async_op=async_op)
        self.grad_handle = h if async_op else True

    def finish_grad_sync(self):
        if self.grad_handle is None:
            self.start_grad_sync()
        if self.grad_handle == "peer":
            peer = self.buf.peer
            if peer["pending"]:
                # the pulls were launched bucket by bucket on the side stream while backward went on: join them
                torch.cuda.current_stream().wait_stream(peer["side"])
                peer["pending"] = False
            peer["pulled"] = True
        elif self.grad_handle is not True and self.grad_handle is not None:
            self.grad_handle.wait()
        if getattr(self, "inter_pending", False):
            # second level: this rank's shard, reduced inside its optimizer instance, is summed across the
            # instances (reference: param_and_grad_buffer.py:405-431)
            buf, b = self.buf, self.bucket
            s, e = buf.shard_range(b)
            op = dist.ReduceOp.AVG if buf.ddp_config.average_in_collective else dist.ReduceOp.SUM
            dist.all_reduce(buf.grad_data[s:e], op=op, group=buf.inter_group)
            self.inter_pending = False
        self.grad_handle = None
        self.ready.clear()
        self.counts.clear()

    def gathers_params(self) -> bool:
        buf = self.buf
        # with peer-memory collectives the optimizer already stored the new weights into every rank
        return buf.use_dist_opt and buf.dp_size > 1 and buf.peer is None

    def _peer_pull(self):
        """Reduce-scatter of this bucket over peer memory, started as soon as the *local* bucket is complete:
        (1) a one-thread kernel on the compute stream tells every peer (a word per bucket and source rank in their
        memory) that this rank's part holds the step's gradients; (2) the pull kernel goes to a side stream behind
        an event, waits in the kernel for the peers' words and then sums the peers' slices of this rank's shard
        (averaging scale fused) on a small grid, while the backward pass keeps the rest of the GPU
        (reference behaviour it replaces: the bucket's asynchronous reduce-scatter,
        megatron/core/distributed/param_and_grad_buffer.py:319-441)."""
        from ..ops.optim import grad_pull_when_ready, peer_signal
        buf, b = self.buf, self.bucket
        peer = buf.peer
        # every rank starts the pull of a bucket exactly once per step, so the count is the same on all of them
        self.pull_count += 1
        dp, me, step = buf.dp_size, buf.dp_rank, self.pull_count
        word = 4 * (b.index * dp + me)
        peer_signal([peer["flag_addr"][q] + word for q in range(dp) if q != me], step)
        # this rank's own word is set on the host side of the same stream (no peer needs to see it)
        peer["flags"][b.index * dp + me:b.index * dp + me + 1].fill_(step)
        cur = torch.cuda.current_stream()
        side = peer["side"]
        side.wait_stream(cur)
        s, e = buf.shard_range(b)
        scale = buf.gradient_scaling_factor * ((1.0 / dp) if buf.ddp_config.average_in_collective else 1.0)
        with torch.cuda.stream(side):
            grad_pull_when_ready([base + 4 * s for base in peer["grad"]], buf.grad_data[s:e], scale,
                                 peer["flags"][b.index * dp:(b.index + 1) * dp], step,
                                 max_blocks=getattr(buf.ddp_config, "peer_pull_blocks", 64))
        peer["pending"] = True

    def start_param_sync(self, force_sync: bool = False):
        """All-gather the updated low-precision shard into the parameter buffer (once per optimizer step)."""
        buf, b = self.buf, self.bucket
        if not self.gathers_params() or not self.params_stale:
            return
        if self.param_handle is not None:
            if force_sync:
                self.param_handle.wait()
                self.param_handle = None
                self.params_stale = False
            return
        s, e = buf.shard_range(b)
        async_op = buf.ddp_config.overlap_param_gather and not force_sync
        h = dist.all_gather_into_tensor(buf.param_data[b.start:b.end], buf.param_data[s:e], group=buf.dp_group,
                                        async_op=async_op)
        if async_op:
            self.param_handle = h
        else:
            self.params_stale = False

    def finish_param_sync(self):
        """Called before the bucket's weights are used.  Waits for the gather in flight, or runs it now when the
        chain has not reached this bucket yet (a module used out of bucket order, evaluation right after a
        step), then starts the next bucket's gather."""
        if self.param_handle is not None:
            self.param_handle.wait()
            self.param_handle = None
            self.params_stale = False
        elif self.params_stale:
            self.start_param_sync(force_sync=True)
        else:
            return
        if self.next_group is not None:            # chain: the gather of the next bucket starts now
            self.next_group.start_param_sync()


class DistributedDataParallel(nn.Module):
    def __init__(self, config: TransformerConfig, ddp_config: DistributedDataParallelConfig, module: nn.Module,
                 disable_bucketing: bool = False):
        super().__init__()
        self.config, self.ddp_config, self.module = config, ddp_config, module
        init = state.model_parallel_is_initialized()
        dp = state.get_data_parallel_world_size(with_context_parallel=True) if init else 1
        if ddp_config.bucket_size is None:
            ddp_config.bucket_size = max(40_000_000, 1_000_000 * dp)
        bucket_size = ddp_config.bucket_size if (ddp_config.overlap_grad_reduce or ddp_config.use_distributed_optimizer) else None
        if getattr(ddp_config, "num_buckets", None):
            # --ddp-num-buckets: a bucket count instead of a bucket size
            total = sum(p.numel() for p in module.parameters() if p.requires_grad)
            bucket_size = max(1, -(-total // int(ddp_config.num_buckets)))
        if disable_bucketing:
            bucket_size = None
        self.bucket_size = bucket_size
        dense, expert = [], []
        for p in module.parameters():
            if not p.requires_grad:
                continue
            (dense if getattr(p, "allreduce", True) else expert).append(p)
        grad_dtype_of = lambda p: torch.float32 if ddp_config.grad_reduce_in_fp32 else p.dtype

        def scaling(dp_size, expert_set):
            if config.calculate_per_token_loss:
                return 1.0
            if ddp_config.average_in_collective:
                if expert_set:
                    return (state.get_expert_data_parallel_world_size() / dp) if init else 1.0
                return 1.0
            return 1.0 / dp

        self.buffers: List[ParamAndGradBuffer] = []
        self.expert_buffers: List[ParamAndGradBuffer] = []
        for plist, is_expert in ((dense, False), (expert, True)):
            groups: Dict[Tuple, List[nn.Parameter]] = {}
            for p in plist:
                groups.setdefault((p.dtype, grad_dtype_of(p)), []).append(p)
            for (pd, gd), ps in groups.items():
                if is_expert:
                    g = state.get_expert_data_parallel_group() if init else None
                    n = state.get_expert_data_parallel_world_size() if init else 1
                    r = state.get_expert_data_parallel_rank() if init else 0
                else:
                    g = state.get_data_parallel_group(with_context_parallel=True) if init else None
                    n, r = dp, (state.get_data_parallel_rank(with_context_parallel=True) if init else 0)
                inter = None
                if not is_expert and init and ddp_config.use_distributed_optimizer and \
                        getattr(ddp_config, "num_distributed_optimizer_instances", 1) > 1:
                    g = state.get_data_parallel_group(with_context_parallel=True, partial_data_parallel=True)
                    n = state.get_data_parallel_world_size(with_context_parallel=True, partial_data_parallel=True)
                    r = state.get_data_parallel_rank(with_context_parallel=True, partial_data_parallel=True)
                    inter = state.get_inter_distributed_optimizer_instance_group()
                buf = ParamAndGradBuffer(ddp_config, ps, pd, gd, g, n, r, bucket_size, scaling(n, is_expert), is_expert,
                                         inter_group=inter)
                (self.expert_buffers if is_expert else self.buffers).append(buf)
        self.bucket_groups: List[BucketGroup] = []
        self.param_to_group: Dict[nn.Parameter, BucketGroup] = {}
        for buf in self.buffers + self.expert_buffers:
            for b in buf.buckets:
                bg = BucketGroup(buf, b)
                self.bucket_groups.append(bg)
                for p in b.params:
                    self.param_to_group[p] = bg
        # parameter gathers are chained in forward order = reverse bucket order, inside each buffer (buffers belong
        # to different optimizers and groups: a chain must not run from the dense weights into the expert weights)
        self.groups_of_buffer: Dict[int, List[BucketGroup]] = {}
        for bg in self.bucket_groups:
            self.groups_of_buffer.setdefault(id(bg.buf), []).append(bg)
        if ddp_config.use_distributed_optimizer and ddp_config.overlap_param_gather:
            for groups in self.groups_of_buffer.values():
                ordered = list(reversed(groups))
                for a, b in zip(ordered[:-1], ordered[1:]):
                    a.next_group = b
        self._install_hooks()
        self._fwd_hooks = []
        if ddp_config.use_distributed_optimizer and ddp_config.overlap_param_gather:
            self._install_forward_pre_hooks()

    # -- readiness ------------------------------------------------------------
    def _install_hooks(self):
        self._accs = []
        for p, bg in self.param_to_group.items():
            p.grad_ready = (lambda p=p, bg=bg: bg.register_grad_ready(p))
            # fallback for gradients produced by plain autograd: fold .grad into main_grad
            acc = p.expand_as(p).grad_fn.next_functions[0][0]

            def hook(*_, p=p, bg=bg):
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None
                    bg.register_grad_ready(p)
            acc.register_hook(hook)
            self._accs.append(acc)

    def _install_forward_pre_hooks(self):
        for m in self.module.modules():
            own = [p for p in m.parameters(recurse=False) if p in self.param_to_group]
            if not own:
                continue

            def pre(mod, args, own=own):
                for p in own:
                    self.param_to_group[p].finish_param_sync()
            self._fwd_hooks.append(m.register_forward_pre_hook(pre))

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    @contextmanager
    def no_sync(self):
        for bg in self.bucket_groups:
            bg.is_last_microbatch = False
        try:
            yield
        finally:
            for bg in self.bucket_groups:
                bg.is_last_microbatch = True

    def start_grad_sync(self, *unused):
        for bg in self.bucket_groups:
            bg.start_grad_sync()

    def finish_grad_sync(self):
        for bg in self.bucket_groups:
            bg.finish_grad_sync()
        # Peer-memory mode: the pulls read the other ranks' gradient buffers in place.  What follows a gradient
        # sync (tensor-parallel all-reduce of sequence-parallel gradients with copy-back, tied-embedding
        # all-reduce, per-token scaling) rewrites those buffers, so nobody may go on before every rank's pulls
        # are done.
        for buf in self.buffers + self.expert_buffers:
            if buf.peer is not None and buf.peer["pulled"]:
                buf.peer["hdl"].barrier()

    def mark_params_updated(self, buffers=None):
        """The optimizer has written new weights into its shards of ``buffers`` (default: all): the other ranks'
        shards in this rank's parameter buffers are out of date until gathered."""
        for buf in (buffers if buffers is not None else self.buffers + self.expert_buffers):
            for bg in self.groups_of_buffer.get(id(buf), []):
                if bg.gathers_params():
                    bg.params_stale = True

    def start_param_sync(self, *unused, force_sync: bool = False, force_dispatch: bool = False, buffers=None):
        """Gather updated weights.  With ``overlap_param_gather`` only the first bucket (in forward order) of each
        buffer is dispatched here; the forward pre-hooks wait for it and chain the rest.  ``force_sync`` gathers
        everything now and waits (before a checkpoint or an evaluation)."""
        for buf in (buffers if buffers is not None else self.buffers + self.expert_buffers):
            groups = self.groups_of_buffer.get(id(buf), [])
            if self.ddp_config.overlap_param_gather and not force_sync:
                if groups:
                    groups[-1].start_param_sync()
            else:
                for bg in groups:
                    bg.start_param_sync(force_sync=True)

    def force_param_sync(self):
        """Every parameter buffer holds the current weights of all ranks when this returns."""
        self.start_param_sync(force_sync=True)

    def scale_gradients(self, factor: float):
        for buf in self.buffers + self.expert_buffers:
            scale_(buf.grad_data, factor)

    def zero_grad_buffer(self):
        for buf in self.buffers + self.expert_buffers:
            buf.zero_grads()
        for bg in self.bucket_groups:
            bg.reset()

    def broadcast_params(self):
        """Make every data-parallel replica start from rank 0's weights."""
        if not (dist.is_initialized() and state.model_parallel_is_initialized()):
            return
        for buf in self.buffers + self.expert_buffers:
            if buf.dp_size > 1:
                src = dist.get_global_rank(buf.dp_group, 0)
                dist.broadcast(buf.param_data, src=src, group=buf.dp_group)

    def state_dict(self, *a, **kw):
        return self.module.state_dict(*a, **kw)

    def load_state_dict(self, sd, strict=True):
        return self.module.load_state_dict(sd, strict=strict)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)
