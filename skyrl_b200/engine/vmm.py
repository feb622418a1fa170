"""Fixed-address device arena (``csrc/vmm_arena.cu``): tensors carved out of it keep their address while the arena
sleeps (physical memory released) and wakes (fresh memory mapped at the same address)."""

from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from ..ops import _lib

_DTYPE_STR = {torch.bfloat16: "<u2", torch.float16: "<f2", torch.float32: "<f4", torch.uint8: "|u1", torch.int32: "<i4"}


class _Span:
    """Raw device memory described through ``__cuda_array_interface__`` (torch wraps it without copying)."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}
        self._owner = owner  # keeps the arena alive as long as a tensor built from this span lives


class VmmArena:
    def __init__(self, nbytes: int, device):
        self.device = torch.device(device)
        lib = _lib.kernels()
        lib.sb_vmm_arena_create.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p),
                                            ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_size_t)]
        for f in (lib.sb_vmm_arena_sleep, lib.sb_vmm_arena_wake, lib.sb_vmm_arena_destroy, lib.sb_vmm_arena_is_mapped):
            f.argtypes = [ctypes.c_void_p]
        h, ptr, size = ctypes.c_void_p(), ctypes.c_ulonglong(), ctypes.c_size_t()
        with torch.cuda.device(self.device):
            code = lib.sb_vmm_arena_create(int(nbytes), ctypes.byref(h), ctypes.byref(ptr), ctypes.byref(size))
        if not h.value:
            _lib.check(code or 2, "sb_vmm_arena_create")
        self._h, self.ptr, self.nbytes = h, int(ptr.value), int(size.value)
        if code != 0:  # reserved but not backed (out of memory): release the range and report
            lib.sb_vmm_arena_destroy(self._h)
            self._h = None
            _lib.check(code, "sb_vmm_arena_create")
        self._off = 0

    def take(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """Next ``shape`` / ``dtype`` tensor of the arena (256-byte aligned; raises when the arena is exhausted)."""
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = (self._off + 255) // 256 * 256
        if off + nbytes > self.nbytes:
            raise MemoryError("arena exhausted")
        self._off = off + nbytes
        raw = torch.as_tensor(_Span(self.ptr + off, nbytes, self), device=self.device)
        return raw.view(dtype).view(*shape)

    @property
    def mapped(self) -> bool:
        return self._h is not None and bool(_lib.kernels().sb_vmm_arena_is_mapped(self._h))

    def sleep(self) -> None:
        torch.cuda.synchronize(self.device)
        _lib.check(_lib.kernels().sb_vmm_arena_sleep(self._h), "sb_vmm_arena_sleep")

    def wake(self, zero: bool = True) -> None:
        with torch.cuda.device(self.device):
            _lib.check(_lib.kernels().sb_vmm_arena_wake(self._h), "sb_vmm_arena_wake")
            if zero:
                torch.as_tensor(_Span(self.ptr, self.nbytes, self), device=self.device).zero_()

    def close(self) -> None:
        if self._h is not None:
            torch.cuda.synchronize(self.device)
            _lib.kernels().sb_vmm_arena_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass
