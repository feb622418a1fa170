"""File IO over local paths and fsspec URLs (``s3://``, ``gs://`` ...): ``open_file``, ``exists``, ``makedirs``,
``local_work_dir`` (work locally, upload on exit) and ``local_read_dir`` (download, read locally)
(reference: skyrl/backends/skyrl_train/utils/io/io.py:22-253)."""

from __future__ import annotations

import contextlib
import os
import shutil
import tempfile
from typing import Iterator, List


def is_remote(path: str) -> bool:
    return "://" in path and not path.startswith("file://")


def _fs(path: str):
    import fsspec

    return fsspec.core.url_to_fs(path)


def open_file(path: str, mode: str = "r", **kw):
    if is_remote(path):
        import fsspec

        return fsspec.open(path, mode, **kw).open()
    if any(c in mode for c in "wax"):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    return open(path, mode, **kw)


def exists(path: str) -> bool:
    if is_remote(path):
        fs, p = _fs(path)
        return fs.exists(p)
    return os.path.exists(path)


def makedirs(path: str, exist_ok: bool = True) -> None:
    if is_remote(path):
        fs, p = _fs(path)
        fs.makedirs(p, exist_ok=exist_ok)
    else:
        os.makedirs(path, exist_ok=exist_ok)


def remove(path: str) -> None:
    if is_remote(path):
        fs, p = _fs(path)
        fs.rm(p, recursive=True)
    elif os.path.isdir(path):
        shutil.rmtree(path, ignore_errors=True)
    elif os.path.exists(path):
        os.remove(path)


def list_dir(path: str) -> List[str]:
    if is_remote(path):
        fs, p = _fs(path)
        return [os.path.basename(x.rstrip("/")) for x in fs.ls(p)]
    return sorted(os.listdir(path))


def upload_directory(local: str, remote: str) -> None:
    fs, p = _fs(remote)
    fs.put(local.rstrip("/") + "/", p.rstrip("/") + "/", recursive=True)


def download_directory(remote: str, local: str) -> None:
    fs, p = _fs(remote)
    fs.get(p.rstrip("/") + "/", local.rstrip("/") + "/", recursive=True)


@contextlib.contextmanager
def local_work_dir(path: str) -> Iterator[str]:
    """Yield a local directory to write into; for remote ``path`` the content is uploaded when the block exits."""
    if not is_remote(path):
        os.makedirs(path, exist_ok=True)
        yield path
        return
    tmp = tempfile.mkdtemp(prefix="skyrl_work_")
    try:
        yield tmp
        upload_directory(tmp, path)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


@contextlib.contextmanager
def local_read_dir(path: str) -> Iterator[str]:
    if not is_remote(path):
        yield path
        return
    tmp = tempfile.mkdtemp(prefix="skyrl_read_")
    try:
        download_directory(path, tmp)
        yield tmp
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def atomic_write_bytes(path: str, data: bytes) -> None:
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
