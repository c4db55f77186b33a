"""Sharded (distributed) checkpoints that can be reloaded under a different TP / PP / DP layout.

Concepts follow the reference's ``dist_checkpointing`` package (mapping.py:50-89 ``ShardedTensor``;
serialization.py:60,310 ``load``/``save``; validation.py:409 integrity check; strategies/
fully_parallel.py:48 spreading replicated shards over data-parallel ranks):

* every tensor of a state dict is described as a hyper-rectangle ``(global_shape, global_offset,
  local_shape)`` of a globally named tensor, optionally narrowed to a ``flattened_range`` of the
  local block (distributed-optimizer shards), with a ``replica_id`` saying which copy is the one to
  write;
* ``save`` writes, per rank, one file with the main-replica blocks it owns plus an index entry per
  block; rank 0 writes the merged index (``metadata.json``) and the non-tensor ``common.pt``;
* ``load`` fills each requested block from every saved block that overlaps it, so the saved and
  the loading layouts need not match.

Two on-disk containers hold the same logical content (keys, global shapes, offsets): the reference's
``torch_dist`` layout (``.metadata`` + ``__<rank>_0.distcp`` + ``common.pt``, written and read by
``checkpoint/torch_dist.py``; the default, so checkpoints interchange with the reference) and a native
one (``metadata.json`` index + ``common.pt`` + one ``shard_<rank>.pt`` per rank).
"""
from __future__ import annotations

import itertools
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.distributed as dist

ReplicaId = Union[int, Tuple[int, ...]]


@dataclass
class ShardedTensor:
    key: str
    data: Optional[torch.Tensor]
    dtype: torch.dtype
    local_shape: Tuple[int, ...]
    global_shape: Tuple[int, ...]
    global_offset: Tuple[int, ...]
    axis_fragmentations: Optional[Tuple[int, ...]] = None
    replica_id: ReplicaId = 0
    prepend_axis_num: int = 0
    allow_shape_mismatch: bool = False
    flattened_range: Optional[slice] = None

    @classmethod
    def from_rank_offsets(cls, key: str, data: torch.Tensor, *rank_offsets: Tuple[int, int, int],
                          replica_id: ReplicaId = 0, prepend_axis_num: int = 0, flattened_range=None,
                          **kw) -> "ShardedTensor":
        """``rank_offsets``: (axis, index of this shard along the axis, number of shards along it).
        Axes below ``prepend_axis_num`` are new leading axes of extent 1 per shard (layer index)."""
        local = (1,) * prepend_axis_num + tuple(data.shape)
        g_shape, g_off, frag = list(local), [0] * len(local), [1] * len(local)
        for axis, idx, n in rank_offsets:
            if not (0 <= idx < n):
                raise ValueError(f"bad rank offset {(axis, idx, n)} for {key}")
            g_shape[axis] = local[axis] * n
            g_off[axis] = local[axis] * idx
            frag[axis] = n
        return cls(key, data, data.dtype, tuple(data.shape), tuple(g_shape), tuple(g_off), tuple(frag), replica_id,
                   prepend_axis_num, flattened_range=flattened_range, **kw)

    def is_main_replica(self) -> bool:
        r = self.replica_id
        return r == 0 if isinstance(r, int) else all(x == 0 for x in r)

    def full_local_shape(self) -> Tuple[int, ...]:
        return (1,) * self.prepend_axis_num + tuple(self.local_shape)

    def without_data(self) -> "ShardedTensor":
        return ShardedTensor(self.key, None, self.dtype, self.local_shape, self.global_shape, self.global_offset,
                             self.axis_fragmentations, self.replica_id, self.prepend_axis_num, self.allow_shape_mismatch,
                             self.flattened_range)

    def validate(self):
        if len(self.global_shape) != len(self.global_offset):
            raise ValueError(f"{self.key}: global shape/offset rank mismatch")
        loc = self.full_local_shape()
        for o, l, g in zip(self.global_offset, loc, self.global_shape):
            if o % max(l, 1) != 0 and not self.allow_shape_mismatch:
                raise ValueError(f"{self.key}: offset {o} is not a multiple of the local extent {l}")
            if o + l > g and not self.allow_shape_mismatch:
                raise ValueError(f"{self.key}: block exceeds the global shape")
        if self.flattened_range is not None and self.data is not None:
            n = self.flattened_range.stop - self.flattened_range.start
            if self.data.numel() != n:
                raise ValueError(f"{self.key}: data has {self.data.numel()} elements, flattened range has {n}")


@dataclass
class ShardedObject:
    """A non-tensor object with a position in a grid of such objects (e.g. per-rank RNG states)."""
    key: str
    data: Any
    global_shape: Tuple[int, ...]
    global_offset: Tuple[int, ...]
    replica_id: ReplicaId = 0

    @property
    def unique_key(self) -> str:
        return f"{self.key}/shard_{'.'.join(map(str, self.global_offset))}_{'.'.join(map(str, self.global_shape))}"

    def is_main_replica(self) -> bool:
        r = self.replica_id
        return r == 0 if isinstance(r, int) else all(x == 0 for x in r)


class LocalNonpersistentObject:
    """State that is never written: on load the locally provided object is returned as is."""

    def __init__(self, obj):
        self.obj = obj

    def unwrap(self):
        return self.obj


# ----------------------------------------------------------------------------- dict walking
def _has_sharded(d) -> bool:
    if isinstance(d, (ShardedTensor, ShardedObject, LocalNonpersistentObject)):
        return True
    if isinstance(d, dict):
        return any(_has_sharded(v) for v in d.values())
    if isinstance(d, (list, tuple)):
        return any(_has_sharded(v) for v in d)
    return False


def _walk(d, prefix=()):
    """Leaves of a nested state dict.  A list/tuple (or dict) without any sharded leaf inside is a
    leaf itself, so plain containers (param groups, args) are saved and restored whole."""
    if isinstance(d, dict) and (prefix == () or _has_sharded(d)):
        for k, v in d.items():
            yield from _walk(v, prefix + (k,))
    elif isinstance(d, (list, tuple)) and _has_sharded(d):
        for i, v in enumerate(d):
            yield from _walk(v, prefix + (i,))
    else:
        yield prefix, d


def _set(d, path, value):
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value


def _to_mutable(d):
    if isinstance(d, dict):
        return {k: _to_mutable(v) for k, v in d.items()}
    if isinstance(d, (list, tuple)):
        return [_to_mutable(v) for v in d]
    return d


def extract_sharded(state_dict):
    """Split a state dict into (sharded tensors, sharded objects, common leaves) by path."""
    tensors, objects, common = [], [], []
    for path, leaf in _walk(state_dict):
        if isinstance(leaf, ShardedTensor):
            tensors.append((path, leaf))
        elif isinstance(leaf, ShardedObject):
            objects.append((path, leaf))
        elif isinstance(leaf, LocalNonpersistentObject):
            continue
        else:
            common.append((path, leaf))
    return tensors, objects, common


# ----------------------------------------------------------------------------- save
def _slices(offset, shape):
    return tuple(slice(o, o + s) for o, s in zip(offset, shape))


def validate_sharding_integrity(index: List[dict]) -> None:
    """Every element of every saved tensor must be covered exactly once by main-replica blocks."""
    by_key: Dict[str, List[dict]] = {}
    for e in index:
        by_key.setdefault(e["key"], []).append(e)
    for key, entries in by_key.items():
        g = tuple(entries[0]["global_shape"])
        total = int(np.prod(g)) if g else 1
        covered = 0
        for e in entries:
            if tuple(e["global_shape"]) != g:
                raise ValueError(f"{key}: inconsistent global shapes {g} vs {tuple(e['global_shape'])}")
            n = int(np.prod(e["local_shape_full"])) if e["local_shape_full"] else 1
            if e["flattened_range"] is not None:
                n = e["flattened_range"][1] - e["flattened_range"][0]
            covered += n
        if covered != total:
            raise ValueError(f"{key}: main replicas cover {covered} of {total} elements")


# Container written by :func:`save`: "torch_dist" = the reference's layout (``.metadata``, ``__<rank>_0.distcp``,
# ``common.pt``; see checkpoint/torch_dist.py), "native" = one ``shard_<rank>.pt`` per rank with a JSON index.
# :func:`load` recognises both.
DEFAULT_CONTAINER = os.environ.get("MLB_CKPT_CONTAINER", "torch_dist")


def save(sharded_state_dict, checkpoint_dir: str, validate_access_integrity: bool = True, group=None,
         container: Optional[str] = None) -> None:
    if (container or DEFAULT_CONTAINER) == "torch_dist":
        from . import torch_dist
        return torch_dist.save(sharded_state_dict, checkpoint_dir, validate_access_integrity, group)
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    os.makedirs(checkpoint_dir, exist_ok=True)
    tensors, objects, common = extract_sharded(sharded_state_dict)
    blobs, index = {}, []
    for _, st in tensors:
        st.validate()
        if not st.is_main_replica():
            continue
        name = f"{st.key}@{'.'.join(map(str, st.global_offset))}" + \
               (f"#{st.flattened_range.start}" if st.flattened_range is not None else "")
        blobs[name] = st.data.detach().cpu().contiguous()
        index.append(dict(key=st.key, blob=name, file=f"shard_{rank}.pt", dtype=str(st.dtype).replace("torch.", ""),
                          global_shape=list(st.global_shape), global_offset=list(st.global_offset),
                          local_shape_full=list(st.full_local_shape()),
                          flattened_range=None if st.flattened_range is None else
                          [st.flattened_range.start, st.flattened_range.stop]))
    objs = {}
    for _, so in objects:
        if so.is_main_replica():
            objs[so.unique_key] = so.data
    torch.save({"tensors": blobs, "objects": objs}, os.path.join(checkpoint_dir, f"shard_{rank}.pt"))
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, (index, list(objs.keys())), group=group)
    else:
        gathered = [(index, list(objs.keys()))]
    if rank == 0:
        full_index = [e for idx, _ in gathered for e in idx]
        obj_index = {k: f"shard_{r}.pt" for r, (_, ks) in enumerate(gathered) for k in ks}
        if validate_access_integrity:
            validate_sharding_integrity(full_index)
        common_sd: Dict = {}
        for path, leaf in common:
            d = common_sd
            for k in path[:-1]:
                d = d.setdefault(k, {})
            d[path[-1]] = leaf
        torch.save(common_sd, os.path.join(checkpoint_dir, "common.pt"))
        with open(os.path.join(checkpoint_dir, "metadata.json"), "w") as f:
            json.dump({"sharded_backend": "mlb_sharded", "sharded_backend_version": 1, "world_size": world,
                       "tensors": full_index, "objects": obj_index}, f)
    if world > 1:
        dist.barrier(group=group)


# ----------------------------------------------------------------------------- load
class _ShardFiles:
    def __init__(self, d):
        self.d, self.cache = d, {}

    def get(self, fname):
        if fname not in self.cache:
            self.cache = {fname: torch.load(os.path.join(self.d, fname), map_location="cpu", weights_only=False)}
        return self.cache[fname]


def _fill(st: ShardedTensor, entries: List[dict], files: Optional[_ShardFiles], strict: bool,
          read_blob=None) -> torch.Tensor:
    """Assemble the block described by ``st`` from the saved blocks overlapping it.  ``read_blob(entry)`` returns
    the saved block of an index entry (default: out of the native shard files)."""
    if read_blob is None:
        read_blob = lambda e: files.get(e["file"])["tensors"][e["blob"]]      # noqa: E731
    full_local = st.full_local_shape()
    want = _slices(st.global_offset, full_local)
    n_want = int(np.prod(full_local)) if full_local else 1
    fr = st.flattened_range
    out = torch.zeros(n_want if fr is None else fr.stop - fr.start, dtype=st.dtype)
    got = 0
    for e in sorted(entries, key=lambda e: e.get("file", "")):
        if tuple(e["global_shape"]) != tuple(st.global_shape) and not st.allow_shape_mismatch:
            raise ValueError(f"{st.key}: checkpoint global shape {e['global_shape']} != requested {st.global_shape}")
        have = _slices(e["global_offset"], e["local_shape_full"])
        inter = []
        for w, h in zip(want, have):
            lo, hi = max(w.start, h.start), min(w.stop, h.stop)
            if lo >= hi:
                inter = None
                break
            inter.append((lo, hi))
        if inter is None:
            continue
        blob = read_blob(e)
        src_shape = tuple(e["local_shape_full"])
        n_src = int(np.prod(src_shape)) if src_shape else 1
        # positions (in the flattened source block) of the intersection, and where they land in the target
        src_idx = torch.arange(n_src).view(src_shape)[tuple(slice(lo - h.start, hi - h.start)
                                                            for (lo, hi), h in zip(inter, have))].reshape(-1)
        dst_idx = torch.arange(n_want).view(full_local)[tuple(slice(lo - w.start, hi - w.start)
                                                              for (lo, hi), w in zip(inter, want))].reshape(-1)
        if e.get("flattened_range") is not None:
            s0, s1 = e["flattened_range"]
            keep = (src_idx >= s0) & (src_idx < s1)
            src_idx, dst_idx = src_idx[keep] - s0, dst_idx[keep]
        if fr is not None:
            keep = (dst_idx >= fr.start) & (dst_idx < fr.stop)
            src_idx, dst_idx = src_idx[keep], dst_idx[keep] - fr.start
        if src_idx.numel() == 0:
            continue
        out[dst_idx] = blob.reshape(-1)[src_idx].to(st.dtype)
        got += src_idx.numel()
    if got != out.numel() and strict:
        raise KeyError(f"{st.key}: only {got} of {out.numel()} requested elements are in the checkpoint")
    return out if fr is not None else out.view(st.local_shape)


def load(sharded_state_dict, checkpoint_dir: str, strict: bool = True, optional_objects: Sequence[str] = ()):
    """Return a plain state dict: every ShardedTensor / ShardedObject leaf replaced by loaded data,
    common (non-sharded) leaves taken from the checkpoint."""
    with open(os.path.join(checkpoint_dir, "metadata.json")) as f:
        meta = json.load(f)
    if meta.get("sharded_backend") == "torch_dist":
        from . import torch_dist
        return torch_dist.load(sharded_state_dict, checkpoint_dir, strict, optional_objects)
    by_key: Dict[str, List[dict]] = {}
    for e in meta["tensors"]:
        by_key.setdefault(e["key"], []).append(e)
    files = _ShardFiles(checkpoint_dir)
    out = _to_mutable(sharded_state_dict)
    tensors, objects, _ = extract_sharded(sharded_state_dict)
    # group by file to keep the shard-file cache effective
    for path, st in tensors:
        if st.key not in by_key:
            if strict:
                raise KeyError(f"tensor {st.key} is not in the checkpoint")
            _set(out, path, st.data)
            continue
        loaded = _fill(st, by_key[st.key], files, strict)
        if st.data is not None:
            st.data.detach().copy_(loaded.view(st.data.shape).to(st.data.device))
            _set(out, path, st.data)
        else:
            _set(out, path, loaded)
    for path, so in objects:
        fname = meta["objects"].get(so.unique_key)
        if fname is None:
            if strict and so.key not in optional_objects:
                raise KeyError(f"object {so.unique_key} is not in the checkpoint")
            _set(out, path, so.data)
            continue
        _set(out, path, files.get(fname)["objects"][so.unique_key])
    for path, leaf in list(_walk(out)):
        if isinstance(leaf, LocalNonpersistentObject):
            _set(out, path, leaf.unwrap())
    common = torch.load(os.path.join(checkpoint_dir, "common.pt"), map_location="cpu", weights_only=False)

    def merge(dst, src):
        for k, v in src.items():
            if isinstance(v, dict) and isinstance(dst.get(k), dict):
                merge(dst[k], v)
            elif k not in dst or not isinstance(dst[k], (torch.Tensor,)):
                dst[k] = v
    if isinstance(out, dict):
        merge(out, common)
    return out


def load_common_state_dict(checkpoint_dir: str):
    return torch.load(os.path.join(checkpoint_dir, "common.pt"), map_location="cpu", weights_only=False)


def load_tensors_metadata(checkpoint_dir: str) -> Dict[str, dict]:
    with open(os.path.join(checkpoint_dir, "metadata.json")) as f:
        meta = json.load(f)
    if meta.get("sharded_backend") == "torch_dist":
        from . import torch_dist
        return torch_dist.load_tensors_metadata(checkpoint_dir)
    return {e["key"]: dict(global_shape=e["global_shape"], dtype=e["dtype"]) for e in meta["tensors"]}


def check_is_distributed_checkpoint(checkpoint_dir: str) -> bool:
    return os.path.isfile(os.path.join(checkpoint_dir, "metadata.json"))


# ----------------------------------------------------------------------------- model -> sharded state dict
def model_sharded_state_dict(model: torch.nn.Module, prefix: str = "", *, tp_rank: int = 0, tp_size: int = 1,
                             dp_rank: int = 0, pp_layer_offset: int = 0, num_layers_global: Optional[int] = None,
                             etp_rank: Optional[int] = None, ep_rank: int = 0, ep_size: int = 1,
                             stack_layers: bool = True) -> Dict[str, ShardedTensor]:
    """Describe every parameter of a model chunk.  Transformer-layer parameters lose their local
    layer index from the key and gain a leading global layer axis (reference:
    transformer_block.py:622-698); TP-sharded parameters are placed along their partition dim;
    a strided partition (gated FC1: [gate; up] per rank) is described as ``stride`` separate
    tensors so that the TP size can change on load (reference: mlp.py:219).  ``stack_layers=False`` is for stacks
    whose layers differ (hybrid Mamba / attention / MLP patterns, dense and expert layers interleaved): a parameter
    that only some layers have cannot fill a layer axis, so each layer keeps its own key with its global index.  So is a parameter whose rows are
    a concatenation of unequal segments (``partition_sizes`` / ``partition_names``: the [z | x | B | C | dt] rows of a
    Mamba mixer's input projection, reference: ssm/mamba_mixer.py ``sharded_state_dict``)."""
    import re
    out: Dict[str, ShardedTensor] = {}
    for name, p in model.state_dict(keep_vars=True).items():
        if not torch.is_tensor(p):
            continue
        key = prefix + name
        offsets = []
        prepend = 0
        m = re.search(r"(^|\.)layers\.(\d+)\.", name)
        if m and num_layers_global is not None and not stack_layers:
            key = prefix + name[:m.start(2)] + str(pp_layer_offset + int(m.group(2))) + name[m.end(2):]
        elif m and num_layers_global is not None:
            local_idx = int(m.group(2))
            key = prefix + name[:m.start(2) - 1 - len("layers")] + "layers." + name[m.end():]
            key = key.replace("..", ".")
            prepend = 1
            offsets.append((0, pp_layer_offset + local_idx, num_layers_global))
        is_tp = bool(getattr(p, "tensor_model_parallel", False)) and tp_size > 1
        replica = (0, 0 if is_tp else tp_rank, dp_rank)
        stride = int(getattr(p, "partition_stride", 1)) if getattr(p, "tensor_model_parallel", False) else 1
        dim = int(getattr(p, "partition_dim", -1))
        data = p.detach()
        sizes = getattr(p, "partition_sizes", None) if getattr(p, "tensor_model_parallel", False) else None
        if (stride > 1 or sizes) and dim >= 0:
            pieces = torch.split(data, list(sizes), dim=dim) if sizes else torch.chunk(data, stride, dim=dim)
            names = getattr(p, "partition_names", None) if sizes else None
            for i, piece in enumerate(pieces):
                off = list(offsets) + ([(dim + prepend, tp_rank, tp_size)] if is_tp else [])
                suffix = names[i] if names else f"part{i}"
                out[f"{name}.part{i}"] = ShardedTensor.from_rank_offsets(f"{key}.{suffix}", piece.contiguous(), *off,
                                                                         replica_id=replica, prepend_axis_num=prepend)
            continue
        if is_tp and dim >= 0:
            offsets.append((dim + prepend, tp_rank, tp_size))
        out[name] = ShardedTensor.from_rank_offsets(key, data, *offsets, replica_id=replica, prepend_axis_num=prepend)
    return out


def load_model_from_sharded(model: torch.nn.Module, loaded: Dict[str, torch.Tensor]) -> None:
    """Copy tensors produced by ``load(model_sharded_state_dict(...))`` back into the module."""
    sd = model.state_dict(keep_vars=True)
    with torch.no_grad():
        for name, p in sd.items():
            if name in loaded:
                p.copy_(loaded[name].view(p.shape).to(p.device))
                continue
            parts = []
            i = 0
            while f"{name}.part{i}" in loaded:
                parts.append(loaded[f"{name}.part{i}"])
                i += 1
            if parts:
                dim = int(getattr(p, "partition_dim", 0))
                p.copy_(torch.cat([t.to(p.device) for t in parts], dim=dim).view(p.shape))


# ----------------------------------------------------------------------------- factories and parallel strategies
@dataclass
class ShardedTensorFactory:
    """A tensor whose on-disk form differs from its in-memory form: ``build_fn(key, data, replica_id)`` turns it
    into a structure of ShardedTensors before saving / loading and ``merge_fn`` turns the loaded structure back
    (reference: dist_checkpointing/mapping.py:606; used e.g. to store a fused [gate; up] weight as two tensors)."""
    key: str
    data: torch.Tensor
    build_fn: Any
    merge_fn: Any
    replica_id: ReplicaId = 0

    def build(self):
        return self.build_fn(self.key, self.data, self.replica_id)


def apply_factories(sharded_state_dict):
    """Replace every factory in place by the structure it builds; returns the factories by path for ``apply_factory_merges``."""
    found = {}

    def walk(d, path=()):
        it = d.items() if isinstance(d, dict) else enumerate(d) if isinstance(d, list) else ()
        for k, v in list(it):
            if isinstance(v, ShardedTensorFactory):
                found[path + (k,)] = v
                d[k] = v.build()
            elif isinstance(v, (dict, list)):
                walk(v, path + (k,))
    walk(sharded_state_dict)
    return found


def apply_factory_merges(loaded_state_dict, factories):
    for path, f in factories.items():
        d = loaded_state_dict
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = f.merge_fn(d[path[-1]])
    return loaded_state_dict


def distribute_main_replicas(sharded_state_dict, group=None):
    """Fully parallel save: shards replicated over the ranks of ``group`` (data-parallel copies) are re-assigned so
    that each is written by exactly one rank and the bytes written per rank are balanced (greedy, largest first;
    reference: strategies/fully_parallel.py:48, exchange_utils.py:121).  Marks the chosen copy ``replica_id = 0``
    and every other copy non-zero; returns the bytes this rank will write."""
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return sum(st.data.numel() * st.data.element_size() for _, st in extract_sharded(sharded_state_dict)[0]
                   if st.is_main_replica())
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    tensors, _, _ = extract_sharded(sharded_state_dict)
    mine = {}
    for _, st in tensors:
        ident = (st.key, tuple(st.global_offset), None if st.flattened_range is None else
                 (st.flattened_range.start, st.flattened_range.stop))
        mine[ident] = st
    sizes = {k: v.data.numel() * v.data.element_size() for k, v in mine.items()}
    gathered = [None] * world
    dist.all_gather_object(gathered, sizes, group=group)
    holders = {}
    for r, d in enumerate(gathered):
        for k, n in d.items():
            holders.setdefault(k, (n, []))[1].append(r)
    load = [0] * world
    owner = {}
    for k, (n, rs) in sorted(holders.items(), key=lambda kv: (-kv[1][0], str(kv[0]))):
        r = min(rs, key=lambda x: (load[x], x))
        owner[k] = r
        load[r] += n
    for k, st in mine.items():
        st.replica_id = 0 if owner[k] == rank else 1
    return load[rank]


def fully_parallel_load(sharded_state_dict, checkpoint_dir: str, group=None, **kw):
    """Fully parallel load: each shard that several ranks of ``group`` need is read from storage by one of them and
    broadcast to the others (reference: strategies/fully_parallel.py:141)."""
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return load(sharded_state_dict, checkpoint_dir, **kw)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    tensors, _, _ = extract_sharded(sharded_state_dict)
    idents = []
    for _, st in tensors:
        idents.append((st.key, tuple(st.global_offset), tuple(st.full_local_shape()),
                       None if st.flattened_range is None else (st.flattened_range.start, st.flattened_range.stop)))
    gathered = [None] * world
    dist.all_gather_object(gathered, idents, group=group)
    same = all(g == gathered[0] for g in gathered)
    if not same:                                    # ranks need different shards: everyone reads its own
        return load(sharded_state_dict, checkpoint_dir, **kw)
    loaded = load(sharded_state_dict, checkpoint_dir, **kw) if rank == 0 else None
    # rank 0 of the group read everything once; the others receive it
    box = [loaded]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0), group=group)
    return box[0]
