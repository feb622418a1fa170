"""Local / cloud storage helpers built on the fsspec utilities: download a checkpoint or dataset to a local cache,
upload a directory (reference: skyrl/utils/storage.py)."""

from __future__ import annotations

import hashlib
import os
from typing import Optional

from . import io as sio


def is_remote(path: str) -> bool:
    return "://" in path and not path.startswith("file://")


def local_cache_path(uri: str, cache_dir: Optional[str] = None) -> str:
    cache_dir = cache_dir or os.path.join(os.path.expanduser("~"), ".cache", "skyrl_b200", "downloads")
    return os.path.join(cache_dir, hashlib.sha256(uri.encode()).hexdigest()[:16], os.path.basename(uri.rstrip("/")))


def download(uri: str, cache_dir: Optional[str] = None, force: bool = False) -> str:
    """Return a local path for ``uri`` (copying remote objects into the cache once)."""
    if not is_remote(uri):
        return os.path.expanduser(uri[7:] if uri.startswith("file://") else uri)
    dst = local_cache_path(uri, cache_dir)
    if os.path.exists(dst) and not force:
        return dst
    os.makedirs(os.path.dirname(dst), exist_ok=True)
    import fsspec

    fs, root = fsspec.core.url_to_fs(uri)
    fs.get(root, dst, recursive=True)
    return dst


def upload_dir(local_dir: str, uri: str) -> None:
    if not is_remote(uri):
        import shutil

        shutil.copytree(local_dir, os.path.expanduser(uri), dirs_exist_ok=True)
        return
    import fsspec

    fs, root = fsspec.core.url_to_fs(uri)
    fs.put(local_dir, root, recursive=True)
