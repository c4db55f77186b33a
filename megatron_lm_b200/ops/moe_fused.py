"""Expert-parallel token dispatch / combine as single kernels over NVLink peer memory.

``FusedMoEComm`` owns, for the expert-parallel group, four symmetric-memory buffers (token rows arriving at
the experts, expert outputs waiting to be pulled, and the two gradient counterparts) and drives the kernels of
``csrc/moe.cu``:

* ``dispatch``  : every routed token copy is stored straight into the receive buffer of the rank that owns its
  expert, in the layout [local expert][source rank][token order] - permute and all-to-all in one launch; the
  receiving rank gets its rows already grouped by expert (no chunk re-sorting);
* ``combine``   : every token pulls its top-k expert outputs from the peers and accumulates them prob-weighted
  in fp32 - all-to-all, un-permute and weighting in one launch.

Backward of dispatch is the pull kernel (sum of the copies' gradients), backward of combine the push kernel
(gradient row scaled by the copy's prob) plus a local dot product for the prob gradient.  The per-expert counts
travel by a small all-gather and are read once on the host (they size the expert GEMM's tile table anyway).
Requires a dropless router (every token has exactly top-k copies).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

_lib.register_signatures({
    "mlb_moe_scatter_rows": "ipppipppiip",
    "mlb_moe_gather_sum": "ipippp" "pp" "iii" "p",
})


def _parr(ptrs: List[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


class FusedMoEComm:
    def __init__(self, group, max_tokens: int, topk: int, hidden: int, num_experts: int, dtype=torch.bfloat16):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.ep, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.E, self.E_local = num_experts, num_experts // self.ep
        self.topk, self.h, self.dtype = topk, hidden, dtype
        self.cap = max_tokens * topk * self.ep                    # worst case: every copy of every rank lands here
        dev = torch.device("cuda", torch.cuda.current_device())
        nbytes = self.cap * hidden * 2
        self.buf = symm_mem.empty(4 * nbytes, dtype=torch.uint8, device=dev)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        base = [int(p) for p in self.hdl.buffer_ptrs]
        self.ptrs = [[b + i * nbytes for b in base] for i in range(4)]     # 0 recv_x, 1 out_y, 2 grad_y, 3 grad_x
        self.views = [self.buf[i * nbytes:(i + 1) * nbytes].view(dtype).view(self.cap, hidden) for i in range(4)]
        self.hdl.barrier()

    def barrier(self):
        self.hdl.barrier()

    # -- routing plan ---------------------------------------------------------------------
    def plan(self, routing_map: torch.Tensor, sorted_indices: torch.Tensor):
        """From the [T, E] routing map and the expert-major copy order: destination (rank, row) of every copy,
        the per-token copy table, and the receive-side counts."""
        dev = routing_map.device
        local_counts = routing_map.sum(dim=0).to(torch.int64)                      # [E]
        all_counts = torch.empty(self.ep, self.E, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(all_counts, local_counts.contiguous(), group=self.group)
        # destination layout on rank d: blocks ordered (local expert, source rank)
        blk = all_counts.view(self.ep, self.ep, self.E_local).permute(1, 2, 0)       # [dst, e_local, src]
        flat = blk.reshape(self.ep, -1)
        offs = torch.cumsum(flat, dim=1) - flat                                    # [dst, e_local * ep]
        my_base = offs.view(self.ep, self.E_local, self.ep)[:, :, self.rank].reshape(-1)   # [E]: base row of my block
        # every token has exactly top-k copies (dropless routing): the number of copies leaving this rank is static
        n_copies = sorted_indices.numel()
        expert_of = torch.repeat_interleave(torch.arange(self.E, device=dev), local_counts, output_size=n_copies)
        start = torch.cumsum(local_counts, 0) - local_counts
        j = torch.arange(n_copies, device=dev) - start[expert_of]
        dst_row = (my_base[expert_of] + j).to(torch.int32)
        dst_rank = (expert_of // self.E_local).to(torch.int32)
        # copies of token t: positions in the expert-major order, grouped by token
        order = torch.argsort(sorted_indices, stable=True)                         # [T * topk]
        # rows per local expert stay on the device (the grouped GEMM builds its tile table there); the only value
        # the host needs is how many rows arrive, to size the activations of the expert MLP: one scalar read
        tpe_local = blk[self.rank].sum(dim=-1)                                       # [E_local] int64, device
        n_recv = int(tpe_local.sum().item())
        return {"dst_rank": dst_rank, "dst_row": dst_row, "order": order.to(torch.int32), "n_copies": n_copies,
                "n_recv": n_recv, "tokens_per_local_expert": tpe_local,
                "src_row": sorted_indices.to(torch.int32)}

    # -- raw kernels ------------------------------------------------------------------------
    def _scatter(self, src, src_row, which: int, dst_rank, dst_row, scale, n):
        _lib.check(_lib.lib().mlb_moe_scatter_rows(_lib.dt(src), src.data_ptr(), _lib.ptr(src_row), _parr(self.ptrs[which]),
                                                   self.ep, dst_rank.data_ptr(), dst_row.data_ptr(), _lib.ptr(scale), n,
                                                   self.h, _lib.stream()), "moe scatter")

    def _gather(self, which: int, src_rank, src_row, weight, out, pulled, n_tokens, k):
        _lib.check(_lib.lib().mlb_moe_gather_sum(_lib.dt(out), _parr(self.ptrs[which]), self.ep, src_rank.data_ptr(),
                                                 src_row.data_ptr(), _lib.ptr(weight), out.data_ptr(), _lib.ptr(pulled),
                                                 n_tokens, k, self.h, _lib.stream()), "moe gather")


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, comm: FusedMoEComm, plan):
        comm.barrier()                                   # peers are done reading the previous contents
        comm._scatter(tokens, plan["src_row"], 0, plan["dst_rank"], plan["dst_row"], None, plan["n_copies"])
        comm.barrier()                                   # every rank's rows have landed
        ctx.comm, ctx.plan, ctx.T = comm, plan, tokens.shape[0]
        return comm.views[0][:plan["n_recv"]].clone()    # the shared buffer is reused by the next layer

    @staticmethod
    def backward(ctx, d_recv):
        comm, plan = ctx.comm, ctx.plan
        comm.barrier()
        comm.views[3][:plan["n_recv"]].copy_(d_recv)
        comm.barrier()
        # gradient of token t = sum of its copies' gradients: gather by the per-token copy table
        o = plan["order"].long()
        out = torch.empty(ctx.T, comm.h, dtype=d_recv.dtype, device=d_recv.device)
        comm._gather(3, plan["dst_rank"][o].contiguous(), plan["dst_row"][o].contiguous(), None, out, None, ctx.T, comm.topk)
        return out, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, copy_probs, comm: FusedMoEComm, plan, T):
        comm.barrier()
        comm.views[1][:plan["n_recv"]].copy_(expert_out)
        comm.barrier()
        o = plan["order"].long()
        src_rank, src_row = plan["dst_rank"][o].contiguous(), plan["dst_row"][o].contiguous()
        w = copy_probs[o].float().contiguous()                                     # [T * topk] grouped by token
        out = torch.empty(T, comm.h, dtype=expert_out.dtype, device=expert_out.device)
        pulled = torch.empty(T * comm.topk, comm.h, dtype=expert_out.dtype, device=expert_out.device)
        comm._gather(1, src_rank, src_row, w, out, pulled, T, comm.topk)
        ctx.save_for_backward(pulled, w, o, src_rank, src_row)
        ctx.comm, ctx.plan, ctx.T, ctx.pdtype = comm, plan, T, copy_probs.dtype
        return out

    @staticmethod
    def backward(ctx, d_out):
        pulled, w, o, src_rank, src_row = ctx.saved_tensors
        comm, plan, T = ctx.comm, ctx.plan, ctx.T
        d_out = d_out.contiguous()
        k = comm.topk
        # prob gradient: <d_out[t], expert output of copy (t, k)>
        dprob_grouped = (pulled.view(T, k, comm.h).float() * d_out.float().unsqueeze(1)).sum(-1).reshape(-1)
        d_copy_probs = torch.empty_like(dprob_grouped)
        d_copy_probs[o] = dprob_grouped
        # expert-output gradient: d_out[t] * prob, pushed to the rank that computed the copy
        comm.barrier()
        tok = torch.arange(T, device=d_out.device, dtype=torch.int32).repeat_interleave(k)
        comm._scatter(d_out, tok, 2, src_rank, src_row, w, T * k)
        comm.barrier()
        d_expert_out = comm.views[2][:plan["n_recv"]].clone()
        return d_expert_out, d_copy_probs.to(ctx.pdtype), None, None, None


def fused_dispatch(tokens, comm, plan):
    return _DispatchFn.apply(tokens.contiguous(), comm, plan)


def fused_combine(expert_out, copy_probs, comm, plan, T):
    return _CombineFn.apply(expert_out.contiguous(), copy_probs, comm, plan, T)
