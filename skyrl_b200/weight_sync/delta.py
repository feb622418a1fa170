"""Delta weight sync through a shared directory: the publisher writes, per weight version, the XOR of every
tensor's bytes against the previous version (compressed; mostly zeros when few bits change) plus a manifest
with checksums; receivers replay deltas onto a local copy of the base checkpoint.

Behavioural reference: skyrl/backends/skyrl_train/weight_sync/{delta_strategy,delta_checkpoint,delta_payload}.py
(``delta-<version:08d>/manifest.json`` + payload files, xxh3-128 checksums, ``write_in_progress`` marker and
reset-from-base on any inconsistency, atomic writes).  Compression uses zlib (the zstd wheel is not in this
image); the codec name is recorded in the manifest so a zstd build can coexist.
"""

from __future__ import annotations

import fcntl
import json
import os
import shutil
import zlib
from typing import Dict, List, Optional

import numpy as np
import torch
import xxhash

from ..models import hf_io
from ..utils.io import atomic_write_bytes

MANIFEST = "manifest.json"


def _delta_dir(root: str, version: int) -> str:
    return os.path.join(root, f"delta-{version:08d}")


def _bytes_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().cpu().view(torch.uint8).reshape(-1).numpy()


def checksum(arr: np.ndarray) -> str:
    return xxhash.xxh3_128_hexdigest(arr.tobytes())


class DeltaPublisher:
    """Trainer side (rank 0): keeps a CPU snapshot of the last published bytes and writes XOR deltas."""

    def __init__(self, sync_dir: str, max_file_bytes: int = 1 << 30, level: int = 1):
        self.sync_dir = sync_dir
        self.max_file_bytes = max_file_bytes
        self.level = level
        self.snapshot: Dict[str, np.ndarray] = {}
        self.version = 0
        os.makedirs(sync_dir, exist_ok=True)

    def publish_base(self, state: Dict[str, torch.Tensor]) -> str:
        """Version 0: a full safetensors checkpoint that receivers copy once."""
        base = os.path.join(self.sync_dir, "base")
        tmp = base + ".tmp"
        os.makedirs(tmp, exist_ok=True)
        hf_io.save_safetensors({k: v.detach().cpu() for k, v in state.items()}, os.path.join(tmp, "model.safetensors"))
        sums = {}
        for k, v in state.items():
            b = _bytes_of(v)
            self.snapshot[k] = b.copy()
            sums[k] = checksum(b)
        atomic_write_bytes(os.path.join(tmp, MANIFEST), json.dumps({"version": 0, "checksums": sums}).encode())
        if os.path.isdir(base):
            shutil.rmtree(base)
        os.replace(tmp, base)
        self.version = 0
        return base

    def publish(self, state: Dict[str, torch.Tensor]) -> str:
        """Write ``delta-<version>`` against the previous publication; returns the directory."""
        if not self.snapshot:
            raise RuntimeError("publish_base() must be called before publish()")
        self.version += 1
        out = _delta_dir(self.sync_dir, self.version)
        tmp = out + ".tmp"
        os.makedirs(tmp, exist_ok=True)
        entries: List[dict] = []
        file_idx, cur, cur_bytes = 0, [], 0

        def flush():
            nonlocal file_idx, cur, cur_bytes
            if not cur:
                return
            fn = f"payload-{file_idx:05d}.bin"
            with open(os.path.join(tmp, fn), "wb") as f:
                off = 0
                for e, blob in cur:
                    e.update(file=fn, offset=off, nbytes=len(blob))
                    f.write(blob)
                    off += len(blob)
            file_idx += 1
            cur, cur_bytes = [], 0

        for name, t in state.items():
            new = _bytes_of(t)
            old = self.snapshot.get(name)
            if old is None or old.shape != new.shape:
                raise ValueError(f"tensor '{name}' changed shape or is new; publish a new base instead")
            patch = np.bitwise_xor(old, new)
            e = {"name": name, "raw_nbytes": int(new.size), "checksum": checksum(new), "changed": bool(patch.any())}
            if e["changed"]:
                blob = zlib.compress(patch.tobytes(), self.level)
                cur.append((e, blob))
                cur_bytes += len(blob)
                if cur_bytes >= self.max_file_bytes:
                    flush()
            entries.append(e)
            self.snapshot[name] = new.copy()
        flush()
        manifest = {"version": self.version, "parent": self.version - 1, "codec": "zlib", "tensors": entries}
        atomic_write_bytes(os.path.join(tmp, MANIFEST), json.dumps(manifest).encode())
        os.replace(tmp, out)
        return out


class LocalCheckpointStore:
    """Receiver side: a local byte copy of the model that deltas are replayed onto, crash-consistently."""

    def __init__(self, sync_dir: str, local_dir: str):
        self.sync_dir, self.local_dir = sync_dir, local_dir
        os.makedirs(local_dir, exist_ok=True)
        self.state_path = os.path.join(local_dir, "store_state.json")
        self.lock_path = os.path.join(local_dir, ".lock")
        self.tensors: Dict[str, np.ndarray] = {}
        self.meta: Dict[str, dict] = {}
        self.version = -1

    # ---- persistent state ---------------------------------------------------------------
    def _read_state(self) -> dict:
        if not os.path.exists(self.state_path):
            return {"version": -1, "write_in_progress": False}
        with open(self.state_path) as f:
            return json.load(f)

    def _write_state(self, version: int, in_progress: bool) -> None:
        atomic_write_bytes(self.state_path, json.dumps({"version": version, "write_in_progress": in_progress}).encode())

    def _lock(self):
        f = open(self.lock_path, "w")
        fcntl.flock(f, fcntl.LOCK_EX)
        return f

    # ---- loading ---------------------------------------------------------------------------
    def reset_from_base(self) -> None:
        base = os.path.join(self.sync_dir, "base")
        header, start = hf_io.read_safetensors_header(os.path.join(base, "model.safetensors"))
        raw = np.fromfile(os.path.join(base, "model.safetensors"), dtype=np.uint8)
        self.tensors, self.meta = {}, {}
        for name, m in header.items():
            if name == "__metadata__":
                continue
            s, e = m["data_offsets"]
            self.tensors[name] = raw[start + s : start + e].copy()
            self.meta[name] = {"dtype": m["dtype"], "shape": m["shape"]}
        with open(os.path.join(base, MANIFEST)) as f:
            sums = json.load(f)["checksums"]
        for name, arr in self.tensors.items():
            if checksum(arr) != sums[name]:
                raise IOError(f"base checkpoint is corrupt: checksum mismatch for '{name}'")
        self.version = 0
        self._persist()

    def _persist(self) -> None:
        self._write_state(self.version, True)
        np.savez(os.path.join(self.local_dir, "tensors.tmp.npz"), **{k.replace("/", "|"): v for k, v in self.tensors.items()})
        os.replace(os.path.join(self.local_dir, "tensors.tmp.npz"), os.path.join(self.local_dir, "tensors.npz"))
        atomic_write_bytes(os.path.join(self.local_dir, "meta.json"), json.dumps(self.meta).encode())
        self._write_state(self.version, False)

    def _load_local(self) -> bool:
        st = self._read_state()
        p = os.path.join(self.local_dir, "tensors.npz")
        if st["write_in_progress"] or st["version"] < 0 or not os.path.exists(p):
            return False
        z = np.load(p)
        self.tensors = {k.replace("|", "/"): z[k] for k in z.files}
        with open(os.path.join(self.local_dir, "meta.json")) as f:
            self.meta = json.load(f)
        self.version = st["version"]
        return True

    # ---- replay ----------------------------------------------------------------------------
    def _apply_one(self, version: int) -> None:
        d = _delta_dir(self.sync_dir, version)
        with open(os.path.join(d, MANIFEST)) as f:
            man = json.load(f)
        if man["parent"] != self.version:
            raise IOError(f"delta {version} expects parent {man['parent']} but the store is at {self.version}")
        files: Dict[str, bytes] = {}
        for e in man["tensors"]:
            if e["changed"]:
                if e["file"] not in files:
                    with open(os.path.join(d, e["file"]), "rb") as f:
                        files[e["file"]] = f.read()
                blob = files[e["file"]][e["offset"] : e["offset"] + e["nbytes"]]
                patch = np.frombuffer(zlib.decompress(blob), dtype=np.uint8)
                if patch.size != e["raw_nbytes"]:
                    raise IOError(f"delta {version}: payload of '{e['name']}' has the wrong size")
                np.bitwise_xor(self.tensors[e["name"]], patch, out=self.tensors[e["name"]])
            if checksum(self.tensors[e["name"]]) != e["checksum"]:
                raise IOError(f"delta {version}: checksum mismatch for '{e['name']}' after replay")
        self.version = version

    def fetch(self, target_version: int) -> int:
        """Bring the local copy to ``target_version``; any inconsistency falls back to a reset from the base."""
        lock = self._lock()
        try:
            if self.version < 0 and not self._load_local():
                self.reset_from_base()
            if self.version > target_version:
                self.reset_from_base()
            try:
                for v in range(self.version + 1, target_version + 1):
                    self._apply_one(v)
            except (IOError, KeyError, zlib.error):
                # purge and replay from the base once
                self.reset_from_base()
                for v in range(1, target_version + 1):
                    self._apply_one(v)
            self._persist()
            return self.version
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
            lock.close()

    def state_dict(self) -> Dict[str, torch.Tensor]:
        out = {}
        for name, arr in self.tensors.items():
            m = self.meta[name]
            out[name] = torch.from_numpy(arr.copy()).view(hf_io._DT[m["dtype"]]).reshape(m["shape"])
        return out
