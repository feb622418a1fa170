"""In-tree build of the native libraries.

Two shared objects are produced under ``skyrl_b200/lib``:

* ``libsb_kernels.so`` -- every ``csrc/*.cu`` file compiled with nvcc for sm_100a only.
* ``libsb_runtime.so`` -- the host-side C++ runtime (``csrc/runtime/*.cpp``: block allocator,
  continuous-batching scheduler, session router hash ring, bin packing).

Both export a plain C ABI and are loaded with ``ctypes`` (see ``skyrl_b200/ops/_lib.py``), so the
build needs neither the PyTorch headers nor a GPU.  ``python -m skyrl_b200.build`` builds everything;
objects are rebuilt only when a source or header is newer than the object.
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return cand


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((CSRC / "runtime").glob("*.h"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _stale(src: Path, obj: Path, hdr_mtime: float) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return src.stat().st_mtime > t or hdr_mtime > t


def _run(cmd: list[str], log: Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd))


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    hdr_mtime = _newest_header_mtime()
    srcs = sorted(CSRC.glob("*.cu"))
    jobs = []
    objs = []
    for src in srcs:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(src, obj, hdr_mtime):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            jobs.append((cmd, OBJ / (src.stem + ".ptxas.log")))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = [ex.submit(_run, cmd, log) for cmd, log in jobs]
            for f in futs:
                f.result()
    out = LIB / "libsb_kernels.so"
    if jobs or not out.exists():
        _run([nvcc, "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    if verbose:
        print(f"[skyrl_b200.build] kernels: {len(jobs)} recompiled -> {out}")
    return out


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    hdr_mtime = _newest_header_mtime()
    srcs = sorted((CSRC / "runtime").glob("*.cpp"))
    out = LIB / "libsb_runtime.so"
    if not srcs:
        return out
    need = force or not out.exists() or any(_stale(s, out, hdr_mtime) for s in srcs)
    if need:
        _run([cxx, *CXX_FLAGS, "-shared", "-o", str(out), *map(str, srcs)])
    if verbose:
        print(f"[skyrl_b200.build] runtime: {'rebuilt' if need else 'up to date'} -> {out}")
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_runtime(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
