"""The reference's ``torch_dist`` on-disk checkpoint layout, written and read directly.

A checkpoint directory holds (reference: megatron/core/dist_checkpointing/strategies/torch.py:648,865 and
serialization.py:310-438):

* ``.metadata``            - pickled ``torch.distributed.checkpoint`` ``Metadata``: for every tensor key its global
                             size, dtype and the list of saved chunks (offsets, sizes); for every chunk where its
                             bytes are (file, offset, length);
* ``__<rank>_0.distcp``    - what rank ``<rank>`` wrote: one ``torch.save`` blob per chunk, back to back; objects
                             (RNG states and the like) as raw pickled bytes under their ``key/shard_<offset>_<shape>``
                             names;
* ``common.pt``            - the replicated, non-sharded part of the state dict (``torch.save``);
* ``metadata.json``        - ``{"sharded_backend": "torch_dist", "sharded_backend_version": 1,
                             "common_backend": "torch", "common_backend_version": 1}``.

Tensor keys, global shapes and offsets are those of the sharded state dict (``checkpoint/sharded.py`` mirrors the
reference's keys, including the prepended layer axis), so model weights interchange with the reference: a
checkpoint written here loads there with ``--no-load-optim`` and one written there loads here.  The chunks are
ordinary N-d blocks; pieces described by a *flattened range* of a block (this framework's distributed-optimizer
state) have no N-d form and are kept beside the files above in the native container (``mlb_flat_<rank>.pt`` with
``mlb_index.json``) - the reference re-expresses such pieces through an internal reformulation that is not part of
the file format.

The files are produced with plain file I/O and ``torch.save`` - no collective planner - so a save needs one
``all_gather_object`` of the chunk tables and nothing else.
"""
from __future__ import annotations

import io
import json
import os
import pickle
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import sharded as ds

_META_JSON = {"sharded_backend": "torch_dist", "sharded_backend_version": 1, "common_backend": "torch",
              "common_backend_version": 1}


def _dcp():
    from torch.distributed.checkpoint import metadata as md
    from torch.distributed.checkpoint.filesystem import _StorageInfo
    return md, _StorageInfo


def is_torch_dist_checkpoint(checkpoint_dir: str) -> bool:
    p = os.path.join(checkpoint_dir, "metadata.json")
    if not (os.path.isfile(p) and os.path.isfile(os.path.join(checkpoint_dir, ".metadata"))):
        return False
    with open(p) as f:
        return json.load(f).get("sharded_backend") == "torch_dist"


# ----------------------------------------------------------------------------- save
def save(sharded_state_dict, checkpoint_dir: str, validate_access_integrity: bool = True, group=None) -> None:
    md, StorageInfo = _dcp()
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    os.makedirs(checkpoint_dir, exist_ok=True)
    tensors, objects, common = ds.extract_sharded(sharded_state_dict)
    fname = f"__{rank}_0.distcp"
    table = []                 # what this rank wrote: dicts with key / kind / placement / storage
    flat_blobs, flat_index = {}, []
    with open(os.path.join(checkpoint_dir, fname), "wb") as f:
        for _, st in tensors:
            st.validate()
            if not st.is_main_replica():
                continue
            if st.flattened_range is not None:
                name = f"{st.key}@{'.'.join(map(str, st.global_offset))}#{st.flattened_range.start}"
                flat_blobs[name] = st.data.detach().cpu().contiguous()
                flat_index.append(dict(key=st.key, blob=name, file=f"mlb_flat_{rank}.pt",
                                       dtype=str(st.dtype).replace("torch.", ""), global_shape=list(st.global_shape),
                                       global_offset=list(st.global_offset), local_shape_full=list(st.full_local_shape()),
                                       flattened_range=[st.flattened_range.start, st.flattened_range.stop]))
                continue
            t = st.data.detach().cpu().contiguous().view(st.full_local_shape())
            off = f.tell()
            torch.save(t, f)
            table.append(dict(key=st.key, kind="tensor", dtype=st.dtype, global_shape=tuple(st.global_shape),
                              offsets=tuple(st.global_offset), sizes=tuple(st.full_local_shape()),
                              storage=(fname, off, f.tell() - off)))
        for _, so in objects:
            if not so.is_main_replica():
                continue
            off = f.tell()
            buf = io.BytesIO()
            torch.save(so.data, buf)
            f.write(buf.getbuffer())
            table.append(dict(key=so.unique_key, kind="bytes", storage=(fname, off, f.tell() - off)))
    if flat_blobs:
        torch.save({"tensors": flat_blobs, "objects": {}}, os.path.join(checkpoint_dir, f"mlb_flat_{rank}.pt"))
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, (table, flat_index), group=group)
    else:
        gathered = [(table, flat_index)]
    if rank == 0:
        sd_meta: Dict[str, Any] = {}
        storage: Dict[Any, Any] = {}
        index_for_check = []
        for tbl, _ in gathered:
            for e in tbl:
                if e["kind"] == "bytes":
                    sd_meta[e["key"]] = md.BytesStorageMetadata()
                    storage[md.MetadataIndex(e["key"])] = StorageInfo(*e["storage"])
                    continue
                tm = sd_meta.get(e["key"])
                if tm is None:
                    tm = md.TensorStorageMetadata(properties=md.TensorProperties(dtype=e["dtype"]),
                                                  size=torch.Size(e["global_shape"]), chunks=[])
                    sd_meta[e["key"]] = tm
                elif tuple(tm.size) != tuple(e["global_shape"]):
                    raise ValueError(f"{e['key']}: ranks disagree on the global shape")
                tm.chunks.append(md.ChunkStorageMetadata(offsets=torch.Size(e["offsets"]), sizes=torch.Size(e["sizes"])))
                storage[md.MetadataIndex(e["key"], torch.Size(e["offsets"]), len(tm.chunks) - 1)] = StorageInfo(*e["storage"])
                index_for_check.append(dict(key=e["key"], global_shape=list(e["global_shape"]),
                                            global_offset=list(e["offsets"]), local_shape_full=list(e["sizes"]),
                                            flattened_range=None))
        flat_all = [e for _, fi in gathered for e in fi]
        if validate_access_integrity:
            ds.validate_sharding_integrity(index_for_check + flat_all)
        meta = md.Metadata(state_dict_metadata=sd_meta, planner_data=None, storage_data=storage)
        try:
            meta.storage_meta = md.StorageMeta(checkpoint_id=checkpoint_dir)
            from torch.distributed.checkpoint.metadata import CURRENT_DCP_VERSION      # noqa: F401
            meta.version = CURRENT_DCP_VERSION
        except Exception:
            pass
        tmp = os.path.join(checkpoint_dir, ".metadata.tmp")
        with open(tmp, "wb") as f:
            pickle.dump(meta, f)
        os.replace(tmp, os.path.join(checkpoint_dir, ".metadata"))
        common_sd: Dict = {}
        for path, leaf in common:
            d = common_sd
            for k in path[:-1]:
                d = d.setdefault(k, {})
            d[path[-1]] = leaf
        torch.save(common_sd, os.path.join(checkpoint_dir, "common.pt"))
        with open(os.path.join(checkpoint_dir, "mlb_index.json"), "w") as f:
            json.dump({"world_size": world, "tensors": flat_all}, f)
        with open(os.path.join(checkpoint_dir, "metadata.json"), "w") as f:
            json.dump(_META_JSON, f)
    if world > 1:
        dist.barrier(group=group)


# ----------------------------------------------------------------------------- load
class _Blobs:
    """Reads chunks out of ``.distcp`` files (one ``torch.load`` per chunk) and flat pieces out of the native files."""

    def __init__(self, d):
        self.d, self.cache = d, {}

    def chunk(self, rel, off, length):
        with open(os.path.join(self.d, rel), "rb") as f:
            f.seek(off)
            return torch.load(io.BytesIO(f.read(length)), map_location="cpu", weights_only=True)

    def obj(self, rel, off, length):
        with open(os.path.join(self.d, rel), "rb") as f:
            f.seek(off)
            return torch.load(io.BytesIO(f.read(length)), map_location="cpu", weights_only=False)

    def flat(self, fname, blob):
        if fname not in self.cache:
            self.cache = {fname: torch.load(os.path.join(self.d, fname), map_location="cpu", weights_only=False)}
        return self.cache[fname]["tensors"][blob]


def load(sharded_state_dict, checkpoint_dir: str, strict: bool = True, optional_objects: Sequence[str] = ()):
    """Same contract as :func:`sharded.load`, for a ``torch_dist`` directory (written here or by the reference)."""
    md, _ = _dcp()
    with open(os.path.join(checkpoint_dir, ".metadata"), "rb") as f:
        meta = pickle.load(f)
    by_key: Dict[str, List[dict]] = {}
    for key, tm in meta.state_dict_metadata.items():
        if not isinstance(tm, md.TensorStorageMetadata):
            continue
        for i, ch in enumerate(tm.chunks):
            info = meta.storage_data[md.MetadataIndex(key, ch.offsets, i)]
            by_key.setdefault(key, []).append(dict(
                key=key, global_shape=list(tm.size), global_offset=list(ch.offsets), local_shape_full=list(ch.sizes),
                flattened_range=None, file=info.relative_path, dcp=(info.relative_path, info.offset, info.length)))
    idx_path = os.path.join(checkpoint_dir, "mlb_index.json")
    if os.path.isfile(idx_path):
        with open(idx_path) as f:
            for e in json.load(f)["tensors"]:
                by_key.setdefault(e["key"], []).append(e)
    blobs = _Blobs(checkpoint_dir)

    def read(e):
        return blobs.chunk(*e["dcp"]) if "dcp" in e else blobs.flat(e["file"], e["blob"])
    out = ds._to_mutable(sharded_state_dict)
    tensors, objects, _ = ds.extract_sharded(sharded_state_dict)
    for path, st in tensors:
        if st.key not in by_key:
            if strict:
                raise KeyError(f"tensor {st.key} is not in the checkpoint")
            ds._set(out, path, st.data)
            continue
        loaded = ds._fill(st, by_key[st.key], None, strict, read_blob=read)
        if st.data is not None:
            st.data.detach().copy_(loaded.view(st.data.shape).to(st.data.device))
            ds._set(out, path, st.data)
        else:
            ds._set(out, path, loaded)
    for path, so in objects:
        tm = meta.state_dict_metadata.get(so.unique_key)
        if tm is None:
            if strict and so.key not in optional_objects:
                raise KeyError(f"object {so.unique_key} is not in the checkpoint")
            ds._set(out, path, so.data)
            continue
        info = meta.storage_data[md.MetadataIndex(so.unique_key)]
        ds._set(out, path, blobs.obj(info.relative_path, info.offset, info.length))
    for path, leaf in list(ds._walk(out)):
        if isinstance(leaf, ds.LocalNonpersistentObject):
            ds._set(out, path, leaf.unwrap())
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


def load_tensors_metadata(checkpoint_dir: str) -> Dict[str, dict]:
    md, _ = _dcp()
    with open(os.path.join(checkpoint_dir, ".metadata"), "rb") as f:
        meta = pickle.load(f)
    return {k: dict(global_shape=list(v.size), dtype=str(v.properties.dtype).replace("torch.", ""))
            for k, v in meta.state_dict_metadata.items() if isinstance(v, md.TensorStorageMetadata)}
