"""Storage back-ends and the LRU cache manager (the reference's ``fs/storage/*.c`` S3 / GCS / Azure API shells,
``fs/cache/cache_manager.c``, ``model_hub/storage/backend.py``).  Object stores share one interface; without network
access the cloud back-ends operate on a local mirror directory, which is also how their tests run."""
from __future__ import annotations

import hashlib
import os
import shutil
from collections import OrderedDict
from typing import List, Optional


class StorageBackend:
    scheme = "file"

    def __init__(self, root: str):
        self.root = os.path.expanduser(root)
        os.makedirs(self.root, exist_ok=True)

    def _p(self, key):
        p = os.path.normpath(os.path.join(self.root, key))
        if not p.startswith(os.path.normpath(self.root)):
            raise ValueError("key escapes the storage root")
        return p

    def put(self, key: str, data: bytes) -> str:
        p = self._p(key)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        tmp = p + ".tmp"
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, p)
        return hashlib.sha256(data).hexdigest()

    def get(self, key: str) -> bytes:
        with open(self._p(key), "rb") as f:
            return f.read()

    def upload_file(self, path: str, key: str):
        p = self._p(key)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        shutil.copyfile(path, p)

    def download_file(self, key: str, path: str):
        shutil.copyfile(self._p(key), path)

    def exists(self, key: str) -> bool:
        return os.path.exists(self._p(key))

    def delete(self, key: str):
        if self.exists(key):
            os.remove(self._p(key))

    def list(self, prefix: str = "") -> List[str]:
        out = []
        for d, _, files in os.walk(self.root):
            for f in files:
                k = os.path.relpath(os.path.join(d, f), self.root)
                if k.startswith(prefix) and not k.endswith(".tmp"):
                    out.append(k)
        return sorted(out)

    def url(self, key: str) -> str:
        return f"{self.scheme}://{key}"


class LocalStorage(StorageBackend):
    pass


class _BucketStorage(StorageBackend):
    def __init__(self, bucket: str, mirror_root: Optional[str] = None, **credentials):
        self.bucket, self.credentials = bucket, credentials
        super().__init__(os.path.join(mirror_root or os.path.expanduser("~/.sneppx/objects"), self.scheme, bucket))

    def url(self, key):
        return f"{self.scheme}://{self.bucket}/{key}"


class S3Storage(_BucketStorage):
    scheme = "s3"


class GCSStorage(_BucketStorage):
    scheme = "gs"


class AzureBlobStorage(_BucketStorage):
    scheme = "az"


def open_storage(url: str, **kw) -> StorageBackend:
    """'s3://bucket', 'gs://bucket', 'az://container' or a local path."""
    for cls in (S3Storage, GCSStorage, AzureBlobStorage):
        if url.startswith(cls.scheme + "://"):
            return cls(url.split("://", 1)[1].strip("/"), **kw)
    return LocalStorage(url)


class CacheManager:
    """Byte-budgeted LRU over named blobs with hit / miss / eviction counters (cache_manager.c)."""

    def __init__(self, capacity_bytes: int):
        self.capacity, self.used = capacity_bytes, 0
        self.items: "OrderedDict[str, bytes]" = OrderedDict()
        self.hits = self.misses = self.evictions = 0

    def get(self, key, loader=None):
        if key in self.items:
            self.items.move_to_end(key)
            self.hits += 1
            return self.items[key]
        self.misses += 1
        if loader is None:
            return None
        val = loader(key)
        self.put(key, val)
        return val

    def put(self, key, val: bytes):
        if key in self.items:
            self.used -= len(self.items.pop(key))
        if len(val) > self.capacity:
            return False
        while self.used + len(val) > self.capacity:
            _, old = self.items.popitem(last=False)
            self.used -= len(old)
            self.evictions += 1
        self.items[key] = val
        self.used += len(val)
        return True

    def stats(self):
        n = self.hits + self.misses
        return {"hits": self.hits, "misses": self.misses, "evictions": self.evictions, "bytes": self.used,
                "hit_rate": self.hits / n if n else 0.0}
