"""Symmetric peer memory: every rank holds device pointers to every other rank's buffers (CUDA IPC over
NVLink), plus the kernel-level collectives built on them (``csrc/comm.cu``).

This replaces, on the hot paths, what the reference delegates to NCCL through FSDP2 / DTensor
(per-parameter ``full_tensor()`` all-gathers in skyrl/backends/skyrl_train/workers/fsdp/fsdp_worker.py:75-128,
reduce-scatter inside ``fully_shard``) and the per-chunk CUDA-IPC handle shuffle of its colocated weight sync
(weight_sync/cuda_ipc_strategy.py:163-258): handles are exchanged once at start-up, after which transfers are
ordinary loads/stores issued from kernels, synchronised by release/acquire flags with bounded waits.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

_cfg_done = False


def _k():
    global _cfg_done
    lib = _lib.kernels()
    if not _cfg_done:
        vp, ci, cl, cf, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_ulonglong
        lib.sb_symm_alloc.argtypes = [u64, ctypes.POINTER(vp)]
        lib.sb_symm_free.argtypes = [vp]
        lib.sb_ipc_get_handle.argtypes = [vp, ctypes.c_char_p]
        lib.sb_ipc_open_handle.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        lib.sb_ipc_close_handle.argtypes = [vp]
        lib.sb_peer_barrier.argtypes = [vp, ci, ci, ci, ci, u64, vp]
        lib.sb_peer_barrier_counter.argtypes = [vp, ci, ci, ci, vp, u64, vp]
        lib.sb_peer_reduce_scatter_f32.argtypes = [vp, ci, cl, cl, vp, vp, vp]
        lib.sb_peer_publish_scalar.argtypes = [vp, ci, ci, vp, vp]
        lib.sb_peer_adamw_push.argtypes = [vp, vp, vp, vp, vp, ci, cl, cl, cf, cf, cf, cf, cf, cf, cf, vp, cf, cf, vp, vp, vp]
        lib.sb_peer_push_bf16.argtypes = [vp, vp, ci, cl, cl, vp]
        lib.sb_peer_push_cast.argtypes = [vp, vp, ci, cl, cl, vp]
        lib.sb_peer_allreduce_bf16.argtypes = [vp, ci, vp, cl, vp]
        _cfg_done = True
    return lib


class _CudaArray:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


@dataclass
class SymmTensor:
    """A local tensor living in a symmetric allocation and the pointers to its twins on the other ranks."""

    local: torch.Tensor
    ptrs: List[int]  # device pointer per rank (own pointer at index rank)

    def ptr_array(self):
        return (ctypes.c_void_p * len(self.ptrs))(*self.ptrs)


def ipc_alloc_tensor(numel: int, dtype: torch.dtype, device: torch.device):
    """A device tensor in its own ``cudaMalloc`` allocation together with the CUDA IPC handle (hex string) through
    which *another process* on the same machine can map it -- e.g. a trainer that pushes weights into a stand-alone
    rollout server's parameter buffer.  Returns ``(tensor, handle_hex, base_pointer)``."""
    nbytes = (numel * torch.empty(0, dtype=dtype).element_size() + 255) // 256 * 256
    p = ctypes.c_void_p()
    _lib.check(_k().sb_symm_alloc(nbytes, ctypes.byref(p)), "sb_symm_alloc")
    buf = ctypes.create_string_buffer(64)
    _lib.check(_k().sb_ipc_get_handle(p, buf), "sb_ipc_get_handle")
    t = torch.as_tensor(_CudaArray(p.value, nbytes), device=device).view(dtype)[:numel]
    return t, bytes(buf.raw).hex(), p.value


def ipc_open(handle_hex: str) -> int:
    """Map another process's allocation (see ``ipc_alloc_tensor``) into this process; returns the device pointer."""
    q = ctypes.c_void_p()
    raw = bytes.fromhex(handle_hex)
    _lib.check(_k().sb_ipc_open_handle(ctypes.create_string_buffer(raw, 64), ctypes.byref(q)), "sb_ipc_open_handle")
    return q.value


class PeerContext:
    def __init__(self, device: torch.device, group: Optional[dist.ProcessGroup] = None, wait_seconds: float = 10.0):
        assert dist.is_initialized(), "PeerContext needs an initialised process group for the handle exchange"
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("peer-memory kernels support up to 8 ranks (one NVSwitch domain)")
        self.device = device
        self.wait_ns = int(wait_seconds * 1e9)
        self._allocs: List[int] = []
        self._opened: List[int] = []
        self._epoch = [0] * 8
        self.signal = self.alloc(8 * 8, torch.int32)  # 8 channels x 8 source slots
        self.norm_pad = self.alloc(8, torch.float32)
        self._sq = torch.zeros(1, device=device, dtype=torch.float32)
        self._norm = torch.zeros(1, device=device, dtype=torch.float32)
        self._skipped = torch.zeros(1, device=device, dtype=torch.int32)
        dist.barrier(group)

    # ------------------------------------------------------------------ memory
    def alloc(self, numel: int, dtype: torch.dtype) -> SymmTensor:
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        nbytes = (nbytes + 255) // 256 * 256
        p = ctypes.c_void_p()
        _lib.check(_k().sb_symm_alloc(nbytes, ctypes.byref(p)), "sb_symm_alloc")
        self._allocs.append(p.value)
        buf = ctypes.create_string_buffer(64)
        _lib.check(_k().sb_ipc_get_handle(p, buf), "sb_ipc_get_handle")
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, bytes(buf.raw), group=self.group)
        ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs.append(p.value)
            else:
                q = ctypes.c_void_p()
                _lib.check(_k().sb_ipc_open_handle(ctypes.create_string_buffer(h, 64), ctypes.byref(q)),
                           "sb_ipc_open_handle")
                self._opened.append(q.value)
                ptrs.append(q.value)
        local = torch.as_tensor(_CudaArray(p.value, nbytes), device=self.device).view(dtype)[:numel]
        return SymmTensor(local, ptrs)

    # ------------------------------------------------------------------ synchronisation
    def barrier(self, channel: int = 0) -> None:
        """Device-side barrier among the ranks, enqueued on the current stream (no host synchronisation)."""
        self._epoch[channel] += 1
        _lib.check(_k().sb_peer_barrier(self.signal.ptr_array(), self.rank, self.world, channel, self._epoch[channel],
                                        self.wait_ns, _lib.stream_ptr()), "sb_peer_barrier")

    def barrier_replayable(self, channel: int) -> None:
        """Device-side barrier whose epoch is kept in device memory, so the launch can be captured in a CUDA graph and
        replayed.  A channel must be used either with this method or with ``barrier``, never with both."""
        if getattr(self, "_epoch_dev", None) is None:
            self._epoch_dev = torch.zeros(8, device=self.device, dtype=torch.int32)
        _lib.check(_k().sb_peer_barrier_counter(self.signal.ptr_array(), self.rank, self.world, channel,
                                                self._epoch_dev[channel:].data_ptr(), self.wait_ns, _lib.stream_ptr()),
                   "sb_peer_barrier_counter")

    # ------------------------------------------------------------------ fused optimizer pieces
    def reduce_scatter_and_norm(self, grads: SymmTensor, out_shard: torch.Tensor, lo: int, n: int) -> None:
        """out_shard = sum over ranks of grads[lo:lo+n]; publishes this shard's squared norm to every rank."""
        self.barrier(0)  # every rank finished writing its gradients
        self._sq.zero_()
        _lib.check(_k().sb_peer_reduce_scatter_f32(grads.ptr_array(), self.world, lo, n, out_shard.data_ptr(),
                                                   self._sq.data_ptr(), _lib.stream_ptr()), "sb_peer_reduce_scatter_f32")
        _lib.check(_k().sb_peer_publish_scalar(self.norm_pad.ptr_array(), self.rank, self.world, self._sq.data_ptr(),
                                               _lib.stream_ptr()), "sb_peer_publish_scalar")
        self.barrier(1)  # all partial norms visible; everyone is done reading everyone's gradients

    BUCKET_CHANNEL = 6

    def reduce_scatter_bucket(self, grads: SymmTensor, out_shard: torch.Tensor, lo: int, n: int, b_lo: int, b_hi: int,
                              first: bool) -> None:
        """Reduce the part of flat range ``[b_lo, b_hi)`` that this rank owns (``[lo, lo + n)``) on the *current* stream:
        a barrier (every rank has finished writing this range's gradients), then loads from every peer.  The squared
        norm accumulates in ``_sq`` across calls (``first`` clears it)."""
        self.barrier(self.BUCKET_CHANNEL)
        if first:
            self._sq.zero_()
        a, b = max(b_lo, lo), min(b_hi, lo + n)
        if b > a:
            _lib.check(_k().sb_peer_reduce_scatter_f32(grads.ptr_array(), self.world, a, b - a, out_shard[a - lo :].data_ptr(),
                                                       self._sq.data_ptr(), _lib.stream_ptr()), "sb_peer_reduce_scatter_f32")

    def finish_reduce(self, grads: SymmTensor, out_shard: torch.Tensor, lo: int, n: int, remaining, first: bool) -> None:
        """Reduce the ranges not covered by ``reduce_scatter_bucket`` calls, then publish the norm partial."""
        self.barrier(0)
        if first:
            self._sq.zero_()
        for (b_lo, b_hi) in remaining:
            a, b = max(b_lo, lo), min(b_hi, lo + n)
            if b > a:
                _lib.check(_k().sb_peer_reduce_scatter_f32(grads.ptr_array(), self.world, a, b - a,
                                                           out_shard[a - lo :].data_ptr(), self._sq.data_ptr(),
                                                           _lib.stream_ptr()), "sb_peer_reduce_scatter_f32")
        _lib.check(_k().sb_peer_publish_scalar(self.norm_pad.ptr_array(), self.rank, self.world, self._sq.data_ptr(),
                                               _lib.stream_ptr()), "sb_peer_publish_scalar")
        self.barrier(1)

    def adamw_and_push(self, master, m, v, grad_shard, params: SymmTensor, lo: int, n: int, lr, beta1, beta2, eps, wd,
                       step: int, max_norm: float, grad_scale: float):
        bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        _lib.check(_k().sb_peer_adamw_push(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad_shard.data_ptr(),
                                           params.ptr_array(), self.world, lo, n, lr, beta1, beta2, eps, wd, bc1, bc2,
                                           self.norm_pad.local.data_ptr(), max_norm, grad_scale, self._norm.data_ptr(),
                                           self._skipped.data_ptr(), _lib.stream_ptr()), "sb_peer_adamw_push")
        self.barrier(2)  # every rank's parameter buffer is complete
        return self._norm, self._skipped

    # ------------------------------------------------------------------ generic transfers
    def push_bf16(self, src: torch.Tensor, dst_ptrs: List[int], dst_offset: int = 0) -> None:
        arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
        if src.dtype == torch.float32:
            _lib.check(_k().sb_peer_push_cast(src.data_ptr(), arr, len(dst_ptrs), dst_offset, src.numel(),
                                              _lib.stream_ptr()), "sb_peer_push_cast")
        else:
            _lib.check(_k().sb_peer_push_bf16(src.data_ptr(), arr, len(dst_ptrs), dst_offset, src.numel(),
                                              _lib.stream_ptr()), "sb_peer_push_bf16")

    def all_reduce_bf16(self, buf: SymmTensor, out: torch.Tensor, n: Optional[int] = None, channel: int = 3) -> torch.Tensor:
        """out = sum over ranks of buf (one-shot: every rank reads every peer). ``buf`` may be reused after return
        of the *next* barrier on ``channel`` (the call brackets the reads with two barriers)."""
        n = n if n is not None else out.numel()
        self.barrier(channel)
        _lib.check(_k().sb_peer_allreduce_bf16(buf.ptr_array(), self.world, out.data_ptr(), n, _lib.stream_ptr()),
                   "sb_peer_allreduce_bf16")
        self.barrier(channel)
        return out

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for q in self._opened:
            _k().sb_ipc_close_handle(ctypes.c_void_p(q))
        self._opened = []
        for p in self._allocs:
            _k().sb_symm_free(ctypes.c_void_p(p))
        self._allocs = []
