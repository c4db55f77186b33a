"""Indexed datasets that live in an object store (``s3://bucket/key`` or ``msc://profile/key`` prefixes).

The small ``.idx`` file is downloaded once into a local cache directory (by the first rank of every node, the
others wait); the ``.bin`` file is read in large ranged chunks that are cached in memory, so consecutive samples
cost one request per ``bin_chunk_nbytes``.

Reference: megatron/core/datasets/object_storage_utils.py (``ObjectStorageConfig`` :21, ``S3Client`` protocol :46,
``is_object_storage_path`` :158, ``get_index_cache_path`` :170, ``parse_s3_path`` :195, ``dataset_exists`` :220,
``cache_index_file`` :243) and the chunked bin readers of indexed_dataset.py (``_S3BinReader`` / ``_MultiStorageClientBinReader``).
The client is whatever a registered factory returns for the scheme: ``boto3`` for ``s3`` and ``multistorageclient``
for ``msc`` when those packages are importable, or any object with the same five methods
(``register_client_factory``); ``LocalDirectoryClient`` serves buckets from a directory tree.
"""
from __future__ import annotations

import os
import shutil
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Protocol, Tuple

import numpy as np

S3_PREFIX = "s3://"
MSC_PREFIX = "msc://"


@dataclass
class ObjectStorageConfig:
    """path_to_idx_cache: local directory for downloaded ``.idx`` files; bin_chunk_nbytes: size of one ranged read."""
    path_to_idx_cache: str
    bin_chunk_nbytes: int = 256 * 1024 * 1024


class ObjectStorageClient(Protocol):
    def download_file(self, Bucket: str, Key: str, Filename: str) -> None: ...
    def upload_file(self, Filename: str, Bucket: str, Key: str) -> None: ...
    def head_object(self, Bucket: str, Key: str) -> Dict[str, Any]: ...
    def get_object(self, Bucket: str, Key: str, Range: str) -> Dict[str, Any]: ...
    def close(self) -> None: ...


class _Body:
    def __init__(self, data: bytes):
        self._data = data

    def read(self) -> bytes:
        return self._data


class LocalDirectoryClient:
    """Buckets are the sub-directories of ``root``; keys are paths below them.  The interface (and the
    ``bytes=a-b`` inclusive range syntax) is that of an S3 client, so the same readers serve both."""

    def __init__(self, root: str):
        self.root = root
        self.requests = 0

    def _path(self, bucket: str, key: str) -> str:
        return os.path.join(self.root, bucket, key)

    def download_file(self, Bucket: str, Key: str, Filename: str) -> None:
        self.requests += 1
        shutil.copyfile(self._path(Bucket, Key), Filename)

    def upload_file(self, Filename: str, Bucket: str, Key: str) -> None:
        dst = self._path(Bucket, Key)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(Filename, dst)

    def head_object(self, Bucket: str, Key: str) -> Dict[str, Any]:
        p = self._path(Bucket, Key)
        if not os.path.isfile(p):
            raise FileNotFoundError(p)
        return {"ContentLength": os.path.getsize(p)}

    def get_object(self, Bucket: str, Key: str, Range: str) -> Dict[str, Any]:
        self.requests += 1
        unit, _, span = Range.partition("=")
        lo, _, hi = span.partition("-")
        if unit != "bytes":
            raise ValueError(f"range {Range!r}")
        with open(self._path(Bucket, Key), "rb") as f:
            f.seek(int(lo))
            return {"Body": _Body(f.read(int(hi) - int(lo) + 1))}

    def close(self) -> None:
        pass


def _boto3_client():
    try:
        import boto3
    except ImportError as e:
        raise RuntimeError("s3:// paths need the boto3 package, or a client registered with "
                           "register_client_factory('s3', ...)") from e
    return boto3.client("s3")


class _MscClient:
    """The five client methods on top of the multi-storage client's file interface (profile = bucket)."""

    def __init__(self, msc):
        self.msc = msc

    def _url(self, bucket, key):
        return f"{MSC_PREFIX}{bucket}/{key}"

    def download_file(self, Bucket, Key, Filename):
        self.msc.download_file(self._url(Bucket, Key), Filename)

    def upload_file(self, Filename, Bucket, Key):
        self.msc.upload_file(self._url(Bucket, Key), Filename)

    def head_object(self, Bucket, Key):
        info = self.msc.info(self._url(Bucket, Key))
        return {"ContentLength": getattr(info, "content_length", None)}

    def get_object(self, Bucket, Key, Range):
        lo, _, hi = Range.partition("=")[2].partition("-")
        with self.msc.open(self._url(Bucket, Key), "rb") as f:
            f.seek(int(lo))
            return {"Body": _Body(f.read(int(hi) - int(lo) + 1))}

    def close(self):
        pass


def _msc_client():
    from ..utils.msc import MultiStorageClientFeature
    try:
        return _MscClient(MultiStorageClientFeature.import_package())
    except RuntimeError as e:
        raise RuntimeError(f"msc:// paths: {e}; or register a client with register_client_factory('msc', ...)") from e


_FACTORIES: Dict[str, Callable[[], ObjectStorageClient]] = {"s3": _boto3_client, "msc": _msc_client}


def register_client_factory(scheme: str, factory: Callable[[], ObjectStorageClient]) -> None:
    _FACTORIES[scheme] = factory


def get_client(path: str) -> ObjectStorageClient:
    return _FACTORIES[get_object_storage_access(path)]()


def is_s3_path(path: str) -> bool:
    return path.startswith(S3_PREFIX)


def is_msc_path(path: str) -> bool:
    return path.startswith(MSC_PREFIX)


def is_object_storage_path(path: str) -> bool:
    return is_s3_path(path) or is_msc_path(path)


def get_object_storage_access(path: str) -> str:
    return "s3" if is_s3_path(path) else "msc"


def parse_s3_path(path: str) -> Tuple[str, str]:
    """``s3://bucket/some/key`` (or ``msc://profile/some/key``) -> (bucket, key)."""
    if not is_object_storage_path(path):
        raise ValueError(f"{path} is not an object-storage path")
    rest = path.split("://", 1)[1]
    bucket, _, key = rest.partition("/")
    if not bucket:
        raise ValueError(f"{path} names no bucket")
    return bucket, key


def get_index_cache_path(idx_path: str, config: ObjectStorageConfig) -> str:
    """Local file that mirrors a remote ``.idx``: the cache directory followed by the path without its scheme."""
    return os.path.join(config.path_to_idx_cache, idx_path.split("://", 1)[1])


def object_exists(client: ObjectStorageClient, path: str) -> bool:
    bucket, key = parse_s3_path(path)
    try:
        client.head_object(Bucket=bucket, Key=key)
        return True
    except Exception as e:                       # a client's "not found" error (404) or a missing file
        code = getattr(e, "response", {}).get("Error", {}).get("Code") if hasattr(e, "response") else None
        if code in (None, "404", "NoSuchKey", "NotFound") or isinstance(e, FileNotFoundError):
            return False
        raise


def dataset_exists(path_prefix: str, idx_path: str, bin_path: str) -> bool:
    client = get_client(path_prefix)
    try:
        return object_exists(client, idx_path) and object_exists(client, bin_path)
    finally:
        client.close()


def cache_index_file(remote_path: str, local_path: str) -> None:
    """Download ``remote_path`` to ``local_path`` once per node: local rank 0 fetches, everybody waits."""
    import torch.distributed as dist
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not os.path.exists(local_path) and (not dist.is_initialized() or local_rank == 0):
        os.makedirs(os.path.dirname(local_path), exist_ok=True)
        client = get_client(remote_path)
        try:
            bucket, key = parse_s3_path(remote_path)
            tmp = f"{local_path}.{os.getpid()}.tmp"
            client.download_file(Bucket=bucket, Key=key, Filename=tmp)
            os.replace(tmp, local_path)
        finally:
            client.close()
    if dist.is_initialized():
        dist.barrier()
    if not os.path.exists(local_path):
        raise FileNotFoundError(f"{local_path} (cached copy of {remote_path})")


class ObjectStorageBinReader:
    """Ranged reads of a remote ``.bin`` through an in-memory chunk: a request inside the cached chunk costs
    nothing, one outside fetches the aligned chunks that cover it."""

    def __init__(self, bin_path: str, config: ObjectStorageConfig, client: Optional[ObjectStorageClient] = None):
        self.bucket, self.key = parse_s3_path(bin_path)
        self.client = client or get_client(bin_path)
        self.chunk = int(config.bin_chunk_nbytes)
        if self.chunk <= 0:
            raise ValueError("bin_chunk_nbytes must be positive")
        self._lo = self._hi = 0
        self._cache: Optional[bytes] = None

    def _fetch(self, lo: int, hi: int) -> bytes:
        return self.client.get_object(Bucket=self.bucket, Key=self.key, Range=f"bytes={lo}-{hi - 1}")["Body"].read()

    def read(self, dtype, count: int, offset: int) -> np.ndarray:
        size = count * np.dtype(dtype).itemsize
        if size == 0:
            return np.empty(0, dtype=dtype)
        if self._cache is not None and self._lo <= offset and offset + size <= self._hi:
            return np.frombuffer(self._cache, dtype=dtype, count=count, offset=offset - self._lo)
        lo = (offset // self.chunk) * self.chunk
        hi = -(-(offset + size) // self.chunk) * self.chunk          # whole chunks: a run of reads never re-fetches
        data = self._fetch(lo, hi)
        self._cache, self._lo, self._hi = data, lo, lo + len(data)
        if offset + size > self._hi:
            raise EOFError(f"{self.key}: read of {size} bytes at {offset} runs past the object's end")
        return np.frombuffer(data, dtype=dtype, count=count, offset=offset - lo)

    def close(self):
        self.client.close()
