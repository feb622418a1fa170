"""ctypes bindings to the in-tree native libraries.

``kernels()`` returns the handle of ``libsb_kernels.so`` (sm_100a CUDA kernels) and ``runtime()`` the
handle of ``libsb_runtime.so`` (host C++ runtime).  On a machine with a CUDA device a missing kernel
library is a hard error: the CUDA path is the product and silently running a PyTorch fallback on a GPU
would hide a broken build.  On CPU-only machines the Python ops use their PyTorch reference
implementations and never ask for the kernel library.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_lock = threading.Lock()
_kernels = None
_runtime = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class NativeLibraryError(RuntimeError):
    pass


def _load(name: str) -> ctypes.CDLL:
    path = _LIB_DIR / name
    if not path.exists():
        if os.environ.get("SKYRL_B200_NO_AUTOBUILD", "0") != "1":
            from skyrl_b200 import build

            build.build_all()
    if not path.exists():
        raise NativeLibraryError(f"{path} is missing; run `python -m skyrl_b200.build`")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


def kernels() -> ctypes.CDLL:
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                lib = _load("libsb_kernels.so")
                lib.sb_version.restype = ctypes.c_char_p
                _kernels = lib
    return _kernels


def runtime() -> ctypes.CDLL:
    global _runtime
    if _runtime is None:
        with _lock:
            if _runtime is None:
                _runtime = _load("libsb_runtime.so")
    return _runtime


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_ERR = {1: "unsupported shape or alignment", 2: "CUDA runtime error", 3: "tensor-map encode failed", 4: "size beyond maximum"}


LAUNCH_COUNT = 0  # kernel-launching library calls made by this process (a call may launch several kernels)
_LAUNCHES_PER_CALL = {"sb_attn_bwd_varlen": 3, "sb_attn_decode_paged": 1}


def check(code: int, what: str) -> None:
    global LAUNCH_COUNT
    LAUNCH_COUNT += _LAUNCHES_PER_CALL.get(what, 1)
    if code != 0:
        raise NativeLibraryError(f"{what} failed: {_ERR.get(code, 'error')} (code {code})")


def status_read_clear() -> int:
    """Device status word: non-zero when a bounded device-side wait gave up. Synchronises."""
    return int(kernels().sb_status_read_clear())


def use_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


# ----------------------------------------------------------------------------- debug-mode index checks
class IndexOutOfRange(NativeLibraryError):
    pass


def debug_bounds() -> bool:
    """``SKYRL_B200_DEBUG_BOUNDS=1``: every op that hands a kernel an index tensor (token ids, cache slots, block
    tables, targets) first checks the indices against the limit the kernel assumes.  Each check synchronises, so this
    is a debugging mode -- the stand-in for running the kernels under a memory checker, which is closed on the shared
    GPU pool.  The kernels themselves do not re-check: an index outside its table is never dereferenced because the
    call raises before the launch."""
    return os.environ.get("SKYRL_B200_DEBUG_BOUNDS", "0") == "1"


def check_index(what: str, idx: torch.Tensor | None, limit: int, min_value: int = 0) -> None:
    """Raise ``IndexOutOfRange`` when any element of ``idx`` lies outside ``[min_value, limit)`` (debug mode only;
    a CUDA-graph capture in progress skips the check because it cannot synchronise)."""
    if idx is None or idx.numel() == 0 or not debug_bounds():
        return
    if idx.is_cuda and torch.cuda.is_current_stream_capturing():
        return
    lo, hi = int(idx.min()), int(idx.max())
    if lo < min_value or hi >= limit:
        raise IndexOutOfRange(f"{what}: index range [{lo}, {hi}] outside [{min_value}, {limit})")


# ----------------------------------------------------------------------------- host<->device accounting
H2D_BYTES = 0
D2H_BYTES = 0


def to_device(t: torch.Tensor, device, non_blocking: bool = True) -> torch.Tensor:
    """Copy a host tensor to ``device`` through pinned memory and account the bytes."""
    global H2D_BYTES
    if torch.device(device).type != "cuda" or t.is_cuda:
        return t.to(device)
    H2D_BYTES += t.numel() * t.element_size()
    if not t.is_pinned():
        t = t.pin_memory()
    return t.to(device, non_blocking=non_blocking)


def to_host(t: torch.Tensor) -> torch.Tensor:
    global D2H_BYTES
    if t.is_cuda:
        D2H_BYTES += t.numel() * t.element_size()
    return t.cpu()
