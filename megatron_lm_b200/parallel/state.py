"""Process-group runtime: the rank grid and every parallel group.

Behavioural contract (reference: megatron/core/parallel_state.py:196-302,
367-442, 468-1186): ranks form a dense grid whose dimension order is given by a
string such as ``"tp-cp-ep-dp-pp"`` with the first token varying fastest; dense
layers see the grid (tp, cp, dp, pp) and expert layers see a second grid
(etp, ep, edp, pp) over the same ranks.  A group for a token set such as
``"tp-dp"`` contains the ranks that differ only in those dimensions.

Design: the grid is a numpy array of rank ids shaped by the order string, and
a group list is obtained by moving the selected axes to the back and reshaping
- there is no per-rank masking arithmetic.  Group objects are created through
``torch.distributed.new_group`` on the chosen backend (NCCL on GPUs, Gloo on
CPU); a "virtual" mode records sizes and ranks without creating communicators
so that sharding metadata and schedules can be unit-tested in one process
(reference test helper: tests/unit_tests/test_utilities.py
``fake_initialize_model_parallel``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist


class RankGrid:
    """Dense N-d grid of ranks; first token of ``order`` varies fastest."""

    def __init__(self, sizes: Dict[str, int], order: str, rank_offset: int = 0):
        self.tokens = [t for t in order.split("-")]
        for t in self.tokens:
            if t not in sizes:
                raise ValueError(f"order token {t!r} has no size")
        for name, n in sizes.items():
            if name not in self.tokens:
                if n != 1:
                    raise ValueError(f"dimension {name} has size {n} but is absent from order {order!r}")
        self.sizes = {t: int(sizes[t]) for t in self.tokens}
        self.world = int(np.prod([self.sizes[t] for t in self.tokens]))
        # numpy is row-major: the LAST axis varies fastest, so reverse the order
        shape = [self.sizes[t] for t in reversed(self.tokens)]
        self.grid = (np.arange(self.world, dtype=np.int64) + rank_offset).reshape(shape)
        self.axis = {t: len(self.tokens) - 1 - i for i, t in enumerate(self.tokens)}

    def groups(self, token: str) -> List[List[int]]:
        """Rank lists of every group spanning the dims named in ``token``.

        Inside a group ranks are ordered with the earlier token of the order
        string varying fastest, and groups are enumerated the same way over the
        remaining dims - this matches the reference enumeration so that group
        creation order (and thus communicator ids) is reproducible."""
        sel = [t for t in self.tokens if t in token.split("-")]
        if not sel:
            return [[int(r)] for r in self.grid.reshape(-1)]
        rest = [t for t in self.tokens if t not in sel]
        # move axes: rest (slow..fast) then sel (slow..fast)
        perm = [self.axis[t] for t in reversed(rest)] + [self.axis[t] for t in reversed(sel)]
        g = np.transpose(self.grid, perm)
        gsize = int(np.prod([self.sizes[t] for t in sel]))
        return g.reshape(-1, gsize).tolist()

    def coords(self, rank: int) -> Dict[str, int]:
        idx = np.argwhere(self.grid == rank)
        if idx.shape[0] != 1:
            raise ValueError(f"rank {rank} not in grid")
        return {t: int(idx[0][self.axis[t]]) for t in self.tokens}


class RankGenerator:
    """Dense + expert grids with the same API shape as the reference's
    ``RankGenerator.get_ranks(token)`` (parallel_state.py:367-442)."""

    def __init__(self, tp: int, ep: int, dp: int, pp: int, cp: int, order: str = "tp-cp-ep-dp-pp",
                 rank_offset: int = 0):
        order = order.lower()
        toks = order.split("-")
        for name, n in (("tp", tp), ("ep", ep), ("dp", dp), ("pp", pp), ("cp", cp)):
            if name not in toks:
                if n != 1:
                    raise RuntimeError(f"size of {name} is {n} but it is missing from order {order}")
                order = order + "-" + name
        self.order = order
        self.tp, self.ep, self.dp, self.pp, self.cp = tp, ep, dp, pp, cp
        self.world_size = tp * dp * pp * cp * ep
        self.grid = RankGrid(dict(tp=tp, ep=ep, dp=dp, pp=pp, cp=cp), order, rank_offset)

    def get_ranks(self, token: str) -> List[List[int]]:
        return self.grid.groups(token)


@dataclass
class _Group:
    name: str
    ranks: List[int]
    size: int
    rank: int                       # rank of this process inside the group
    pg: Optional[object] = None     # torch ProcessGroup (None in virtual mode / size 1 w/o comm)
    gloo_pg: Optional[object] = None


@dataclass
class _State:
    initialized: bool = False
    virtual: bool = False
    world_size: int = 1
    rank: int = 0
    groups: Dict[str, _Group] = field(default_factory=dict)
    all_group_ranks: Dict[str, List[List[int]]] = field(default_factory=dict)
    vpp_size: Optional[int] = None
    vpp_rank: Optional[int] = None
    order: str = "tp-cp-ep-dp-pp"
    embedding_ranks: List[int] = field(default_factory=list)
    position_embedding_ranks: List[int] = field(default_factory=list)
    memory_buffer: Optional[object] = None
    nccl_cfg: Optional[dict] = None
    pp_channels: Optional[dict] = None


_S = _State()


def _nccl_options(name: str, cfg: Optional[dict], high_priority: Sequence[str] = ()):
    """Per-group NCCL tuning (reference: parallel_state.py:131-163)."""
    if not (dist.is_available() and dist.is_nccl_available()):
        return None
    entry = (cfg or {}).get(name)
    if entry is None and name not in high_priority:
        return None
    opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=name in high_priority)
    if entry:
        for key in ("cga_cluster_size", "max_ctas", "min_ctas"):
            if key in entry:
                setattr(opts.config, key, entry[key])
        if "net_name" in entry:
            opts.config.net_name = entry["net_name"]
    return opts


def _make(name: str, rank_lists: List[List[int]], *, backend=None, gloo_twin=False, timeout=None,
          pg_options=None):
    """Create every communicator of one kind (all ranks must call) and remember ours."""
    _S.all_group_ranks[name] = rank_lists
    mine = None
    for ranks in rank_lists:
        pg = gpg = None
        if not _S.virtual and dist.is_initialized():
            kw = {}
            if timeout is not None:
                kw["timeout"] = timeout
            if pg_options is not None:
                kw["pg_options"] = pg_options
            pg = dist.new_group(ranks, backend=backend, **kw)
            if gloo_twin:
                gpg = dist.new_group(ranks, backend="gloo", **({"timeout": timeout} if timeout else {}))
        if _S.rank in ranks:
            mine = _Group(name, list(ranks), len(ranks), ranks.index(_S.rank), pg, gpg)
    if mine is None:
        raise RuntimeError(f"rank {_S.rank} is in no {name} group")
    _S.groups[name] = mine


def initialize_model_parallel(
    tensor_model_parallel_size: int = 1,
    pipeline_model_parallel_size: int = 1,
    virtual_pipeline_model_parallel_size: Optional[int] = None,
    pipeline_model_parallel_comm_backend: Optional[str] = None,
    use_sharp: bool = False,
    context_parallel_size: int = 1,
    hierarchical_context_parallel_sizes: Optional[List[int]] = None,
    expert_model_parallel_size: int = 1,
    num_distributed_optimizer_instances: int = 1,
    expert_tensor_parallel_size: Optional[int] = None,
    nccl_communicator_config_path: Optional[str] = None,
    distributed_timeout_minutes: int = 30,
    order: str = "tp-cp-ep-dp-pp",
    create_gloo_process_groups: bool = True,
    high_priority_stream_groups: Sequence[str] = (),
    *,
    virtual: bool = False,
    virtual_world_size: Optional[int] = None,
    virtual_rank: int = 0,
) -> None:
    """Build every parallel group (reference: parallel_state.py:468-1186).

    With ``virtual=True`` nothing is communicated: the sizes and this
    process's would-be rank in each group are recorded for ``virtual_rank`` in
    a world of ``virtual_world_size``."""
    if _S.initialized:
        raise RuntimeError("model parallel is already initialized")
    if virtual:
        world, rank = int(virtual_world_size or 1), int(virtual_rank)
    else:
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialized")
        world, rank = dist.get_world_size(), dist.get_rank()
    tp, pp, cp, ep = (tensor_model_parallel_size, pipeline_model_parallel_size,
                      context_parallel_size, expert_model_parallel_size)
    model_size = tp * pp * cp
    if world % model_size != 0:
        raise RuntimeError(f"world_size ({world}) is not divisible by tp*pp*cp ({model_size})")
    dp = world // model_size
    etp = expert_tensor_parallel_size if expert_tensor_parallel_size is not None else tp
    expert_model_size = etp * ep * pp
    if world % expert_model_size != 0:
        raise RuntimeError(f"world_size ({world}) is not divisible by etp*ep*pp ({expert_model_size})")
    edp = world // expert_model_size
    if virtual_pipeline_model_parallel_size is not None and pp <= 1 and virtual_pipeline_model_parallel_size > 1:
        raise RuntimeError("virtual pipeline needs pipeline_model_parallel_size > 1")
    if dp % num_distributed_optimizer_instances != 0:
        raise RuntimeError("dp size must be divisible by num_distributed_optimizer_instances")

    _S.virtual, _S.world_size, _S.rank, _S.order = virtual, world, rank, order
    _S.vpp_size = virtual_pipeline_model_parallel_size
    _S.vpp_rank = 0 if virtual_pipeline_model_parallel_size is not None else None
    if nccl_communicator_config_path:
        import yaml
        with open(nccl_communicator_config_path) as f:
            _S.nccl_cfg = yaml.safe_load(f)
    timeout = timedelta(minutes=distributed_timeout_minutes)
    backend = None
    if not virtual:
        backend = dist.get_backend()
    is_nccl = backend == "nccl"
    gloo = create_gloo_process_groups and not virtual and is_nccl

    dense = RankGenerator(tp=tp, ep=1, dp=dp, pp=pp, cp=cp, order=order)
    expert = RankGenerator(tp=etp, ep=ep, dp=edp, pp=pp, cp=1, order=order)
    # the two decompositions must agree on pipeline stages
    if dense.get_ranks("pp") != expert.get_ranks("pp"):
        raise RuntimeError("dense and expert grids disagree on pipeline groups")

    def mk(name, token, gen=dense, twin=False):
        opts = _nccl_options(name, _S.nccl_cfg, high_priority_stream_groups) if is_nccl else None
        _make(name, gen.get_ranks(token), backend=backend, gloo_twin=twin and gloo, timeout=timeout,
              pg_options=opts)

    mk("dp", "dp", twin=True)
    mk("dp_cp", "dp-cp", twin=True)
    # partial-DP groups for multiple distributed-optimizer instances
    if num_distributed_optimizer_instances > 1:
        inst = dp * cp // num_distributed_optimizer_instances
        intra, inter = [], []
        for ranks in dense.get_ranks("dp-cp"):
            for i in range(num_distributed_optimizer_instances):
                intra.append(ranks[i * inst:(i + 1) * inst])
            for j in range(inst):
                inter.append(ranks[j::inst])
        _make("intra_dp_cp", intra, backend=backend, gloo_twin=gloo, timeout=timeout)
        _make("inter_dp_cp", inter, backend=backend, timeout=timeout)
    else:
        _S.all_group_ranks["intra_dp_cp"] = _S.all_group_ranks["dp_cp"]
        _S.groups["intra_dp_cp"] = _S.groups["dp_cp"]
    mk("cp", "cp")
    if hierarchical_context_parallel_sizes:
        if int(np.prod(hierarchical_context_parallel_sizes)) != cp:
            raise RuntimeError("hierarchical_context_parallel_sizes must multiply to cp")
        # level 0 is the innermost (fastest varying) sub-group
        for lvl, _ in enumerate(hierarchical_context_parallel_sizes):
            lists = []
            for ranks in dense.get_ranks("cp"):
                arr = np.array(ranks).reshape(list(reversed(hierarchical_context_parallel_sizes)))
                ax = len(hierarchical_context_parallel_sizes) - 1 - lvl
                lists += np.moveaxis(arr, ax, -1).reshape(-1, arr.shape[ax]).tolist()
            _make(f"hcp{lvl}", lists, backend=backend, timeout=timeout)
    mk("mp", "tp-pp")
    mk("tp", "tp")
    pp_backend = pipeline_model_parallel_comm_backend or backend
    _make("pp", dense.get_ranks("pp"), backend=pp_backend if not virtual else None, timeout=timeout)
    # one-directional pipeline channels.  Every (sender stage -> receiver stage, activation or gradient) stream of
    # messages gets a communicator of its own, so each communicator carries a strict FIFO from one sender to one
    # receiver.  NCCL runs the point-to-point kernels of one communicator in issue order on one stream; with sends
    # and receives of both directions mixed on one communicator, two stages that each post a receive before their
    # send (or two sends first) would wait on each other for ever.  With one channel per direction and kind that
    # cannot happen, whatever order the schedule posts its transfers in.
    _S.pp_channels = {}
    # A posted receive is a kernel that spins until the neighbour stage sends, i.e. for as long as that stage
    # computes; it holds one SM per NCCL channel all that time.  Activations of one microbatch are a few MB, so two
    # channels are plenty and leave the SMs to the GEMMs ("pp_channel" in the NCCL config overrides this).
    ch_opts = None
    if is_nccl and pp_backend == "nccl":
        cfg_ch = dict(_S.nccl_cfg or {})
        cfg_ch.setdefault("pp_channel", {"max_ctas": 2, "min_ctas": 1})
        ch_opts = _nccl_options("pp_channel", cfg_ch)
    if pp > 1:
        for ranks in dense.get_ranks("pp"):
            for s in range(len(ranks)):
                pair = sorted({ranks[s], ranks[(s + 1) % len(ranks)]})
                for kind in ("F", "B"):
                    pg = None
                    if not virtual and dist.is_initialized():
                        try:
                            pg = dist.new_group(pair, backend=pp_backend, timeout=timeout,
                                                **({"pg_options": ch_opts} if ch_opts is not None else {}))
                        except (RuntimeError, TypeError, ValueError):
                            # a build of the collective library that does not take the channel cap: default options
                            ch_opts = None
                            pg = dist.new_group(pair, backend=pp_backend, timeout=timeout)
                    if rank in ranks and rank in pair:
                        _S.pp_channels[(kind, s)] = pg
    # embedding groups: first and last pipeline stage (tied embeddings)
    emb, pos = [], []
    for ranks in dense.get_ranks("pp"):
        e = [ranks[0]] if len(ranks) == 1 else [ranks[0], ranks[-1]]
        emb.append(e)
        pos.append([ranks[0]])
    _S.all_group_ranks["embd"] = emb
    _S.all_group_ranks["pos_embd"] = pos
    for name, lists in (("embd", emb), ("pos_embd", pos)):
        mine = None
        for ranks in lists:
            pg = None
            if not virtual and dist.is_initialized():
                pg = dist.new_group(ranks, backend=backend, timeout=timeout)
            if rank in ranks:
                mine = _Group(name, ranks, len(ranks), ranks.index(rank), pg)
        if mine is not None:
            _S.groups[name] = mine
    mk("tp_dp_cp", "tp-dp-cp")
    mk("tp_dp", "tp-dp")
    mk("tp_cp", "tp-cp")
    # expert grid
    mk("ep", "ep", gen=expert)
    mk("etp", "tp", gen=expert)
    mk("tp_ep", "tp-ep", gen=expert)
    mk("tp_ep_pp", "tp-ep-pp", gen=expert)
    mk("edp", "dp", gen=expert, twin=True)
    _S.initialized = True
    from ..utils.memory import GlobalMemoryBuffer
    _S.memory_buffer = GlobalMemoryBuffer()


def fake_initialize_model_parallel(world_size: int, rank: int = 0, **kw) -> None:
    """Virtual ranks without communicators (single-process unit tests)."""
    initialize_model_parallel(virtual=True, virtual_world_size=world_size, virtual_rank=rank, **kw)


def model_parallel_is_initialized() -> bool:
    return _S.initialized


def destroy_model_parallel() -> None:
    global _S
    if _S.initialized and not _S.virtual and dist.is_initialized():
        seen = set()
        for g in _S.groups.values():
            for pg in (g.pg, g.gloo_pg):
                if pg is not None and id(pg) not in seen:
                    seen.add(id(pg))
                    try:
                        dist.destroy_process_group(pg)
                    except Exception:
                        pass
        for pg in (_S.pp_channels or {}).values():
            if pg is not None:
                try:
                    dist.destroy_process_group(pg)
                except Exception:
                    pass
    _S = _State()


# --------------------------------------------------------------------- getters
def _g(name: str) -> _Group:
    if not _S.initialized:
        raise RuntimeError("model parallel is not initialized")
    if name not in _S.groups:
        raise RuntimeError(f"this rank is not part of a {name} group")
    return _S.groups[name]


def get_group(name: str):
    return _g(name).pg


def get_group_ranks(name: str) -> List[int]:
    return list(_g(name).ranks)


def get_all_group_ranks(name: str) -> List[List[int]]:
    return _S.all_group_ranks[name]


def get_group_size(name: str) -> int:
    return _g(name).size if _S.initialized else 1


def get_group_rank(name: str) -> int:
    return _g(name).rank if _S.initialized else 0


# reference-named getters (parallel_state.py:1189-1850)
def get_tensor_model_parallel_group(): return _g("tp").pg
def get_tensor_model_parallel_world_size(): return get_group_size("tp")
def get_tensor_model_parallel_rank(): return get_group_rank("tp")
def get_tensor_model_parallel_src_rank(): return _g("tp").ranks[0]
def get_pipeline_model_parallel_group(): return _g("pp").pg


def get_pipeline_channel(kind: str, sender_stage: int):
    """Communicator of one one-directional pipeline channel: ``("F", s)`` carries activations from stage ``s`` to
    stage ``s + 1`` (wrapping), ``("B", s)`` carries gradients from stage ``s + 1`` back to stage ``s``.  None when
    this rank is on neither end (or pipeline parallelism is off)."""
    return (_S.pp_channels or {}).get((kind, sender_stage))


def get_pipeline_model_parallel_world_size(): return get_group_size("pp")
def get_pipeline_model_parallel_rank(): return get_group_rank("pp")
def get_model_parallel_group(): return _g("mp").pg
def get_context_parallel_group(): return _g("cp").pg
def get_context_parallel_world_size(): return get_group_size("cp")
def get_context_parallel_rank(): return get_group_rank("cp")
def get_context_parallel_global_ranks(): return get_group_ranks("cp")
def get_hierarchical_context_parallel_groups(): return [g.pg for n, g in sorted(_S.groups.items()) if n.startswith("hcp")]
def get_expert_model_parallel_group(): return _g("ep").pg
def get_expert_model_parallel_world_size(): return get_group_size("ep")
def get_expert_model_parallel_rank(): return get_group_rank("ep")
def get_expert_tensor_parallel_group(): return _g("etp").pg
def get_expert_tensor_parallel_world_size(): return get_group_size("etp")
def get_expert_tensor_parallel_rank(): return get_group_rank("etp")
def get_expert_tensor_and_model_parallel_group(): return _g("tp_ep").pg
def get_expert_tensor_and_model_parallel_world_size(): return get_group_size("tp_ep")
def get_expert_tensor_model_pipeline_parallel_group(): return _g("tp_ep_pp").pg
def get_expert_data_parallel_group(): return _g("edp").pg
def get_expert_data_parallel_world_size(): return get_group_size("edp")
def get_expert_data_parallel_rank(): return get_group_rank("edp")
def get_expert_data_parallel_group_gloo(): return _g("edp").gloo_pg
def get_tensor_and_data_parallel_group(with_context_parallel=False):
    return _g("tp_dp_cp" if with_context_parallel else "tp_dp").pg
def get_tensor_and_context_parallel_group(): return _g("tp_cp").pg
def get_embedding_group(): return _S.groups["embd"].pg if "embd" in _S.groups else None
def get_position_embedding_group(): return _S.groups["pos_embd"].pg if "pos_embd" in _S.groups else None
def get_amax_reduction_group(with_context_parallel=False, tp_only_amax_red=False):
    if tp_only_amax_red:
        return _g("tp").pg
    return _g("tp_dp_cp" if with_context_parallel else "tp_dp").pg


def get_data_parallel_group(with_context_parallel=False, partial_data_parallel=False):
    if partial_data_parallel:
        return _g("intra_dp_cp").pg
    return _g("dp_cp" if with_context_parallel else "dp").pg


def get_data_parallel_group_gloo(with_context_parallel=False, partial_data_parallel=False):
    if partial_data_parallel:
        return _g("intra_dp_cp").gloo_pg
    return _g("dp_cp" if with_context_parallel else "dp").gloo_pg


def get_inter_distributed_optimizer_instance_group():
    return _g("inter_dp_cp").pg


def get_data_parallel_world_size(with_context_parallel=False, partial_data_parallel=False):
    if not _S.initialized:
        return 1
    if partial_data_parallel:
        return _g("intra_dp_cp").size
    return _g("dp_cp" if with_context_parallel else "dp").size


def get_data_parallel_rank(with_context_parallel=False, partial_data_parallel=False):
    if not _S.initialized:
        return 0
    if partial_data_parallel:
        return _g("intra_dp_cp").rank
    return _g("dp_cp" if with_context_parallel else "dp").rank


def get_data_parallel_src_rank(with_context_parallel=False):
    return _g("dp_cp" if with_context_parallel else "dp").ranks[0]


def get_virtual_pipeline_model_parallel_world_size(): return _S.vpp_size
def get_virtual_pipeline_model_parallel_rank(): return _S.vpp_rank


def set_virtual_pipeline_model_parallel_rank(r: Optional[int]) -> None:
    _S.vpp_rank = r


def is_pipeline_first_stage(ignore_virtual: bool = True, vp_stage: Optional[int] = None) -> bool:
    if not ignore_virtual and _S.vpp_size is not None:
        v = _S.vpp_rank if vp_stage is None else vp_stage
        if v != 0:
            return False
    return get_pipeline_model_parallel_rank() == 0


def is_pipeline_last_stage(ignore_virtual: bool = True, vp_stage: Optional[int] = None) -> bool:
    if not ignore_virtual and _S.vpp_size is not None:
        v = _S.vpp_rank if vp_stage is None else vp_stage
        if v != _S.vpp_size - 1:
            return False
    return get_pipeline_model_parallel_rank() == get_pipeline_model_parallel_world_size() - 1


def is_rank_in_embedding_group(ignore_virtual: bool = True, vp_stage: Optional[int] = None) -> bool:
    if "embd" not in _S.groups:
        return False
    ranks = _S.groups["embd"].ranks
    if ignore_virtual or _S.vpp_size is None:
        return _S.rank in ranks
    if _S.rank == ranks[0]:
        return is_pipeline_first_stage(ignore_virtual=False, vp_stage=vp_stage)
    if _S.rank == ranks[-1]:
        return is_pipeline_last_stage(ignore_virtual=False, vp_stage=vp_stage)
    return False


def is_rank_in_position_embedding_group() -> bool:
    return "pos_embd" in _S.groups


def get_pipeline_model_parallel_first_rank(): return _g("pp").ranks[0]
def get_pipeline_model_parallel_last_rank(): return _g("pp").ranks[-1]


def get_pipeline_model_parallel_next_rank():
    g = _g("pp")
    return g.ranks[(g.rank + 1) % g.size]


def get_pipeline_model_parallel_prev_rank():
    g = _g("pp")
    return g.ranks[(g.rank - 1) % g.size]


def get_global_memory_buffer():
    return _S.memory_buffer


def get_rank() -> int:
    return _S.rank if _S.initialized else (dist.get_rank() if dist.is_initialized() else 0)


def get_world_size() -> int:
    return _S.world_size if _S.initialized else (dist.get_world_size() if dist.is_initialized() else 1)
