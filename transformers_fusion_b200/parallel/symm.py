"""Symmetric peer memory: buffers that exist at the same logical place on every GPU of the node and
can be read / written by any rank's kernels over NVLink.

Each rank allocates with cudaMalloc inside the kernel library, exports a CUDA IPC handle, and the
handles are exchanged through ``torch.distributed`` (the control plane); the data plane is the
kernels' own peer loads and stores.  ``SymmBuffer.ptrs`` is a device int64 tensor with the W base
addresses (slot ``rank`` is the local one), ready to be handed to a kernel.

Reference counterpart: the process-local shared vectors of DistributedContext
(src/trainer/distributed.cpp:21-25) — here real cross-process GPU memory.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib

_lib.register("tfb_comm_barrier", [_lib.c_p, _lib.c_p, _lib.c_i, _lib.c_i, _lib.c_p, _lib.c_p])


class _RawCuda:
    """Zero-copy view of a raw device allocation through __cuda_array_interface__."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class SymmBuffer:
    def __init__(self, heap, nbytes, local_ptr, peer_ptrs):
        self.heap, self.nbytes, self.local_ptr, self.peer_ptrs = heap, nbytes, local_ptr, peer_ptrs
        self.bytes = torch.as_tensor(_RawCuda(local_ptr, nbytes), device=heap.device)
        self.ptrs = torch.tensor(peer_ptrs, dtype=torch.int64, device=heap.device)

    def view(self, dtype, numel=None):
        t = self.bytes.view(dtype)
        return t if numel is None else t[:numel]


class SymmetricHeap:
    def __init__(self, rank: int, world: int, device, group=None):
        self.rank, self.world, self.device, self.group = rank, world, torch.device(device), group
        self.buffers = []
        self._reset_hooks = []
        lib = _lib.lib()
        for name in ("tfb_symm_alloc", "tfb_symm_open", "tfb_symm_close", "tfb_symm_free"):
            getattr(lib, name).restype = C.c_int
        lib.tfb_symm_alloc.argtypes = [C.c_longlong, C.POINTER(C.c_void_p), C.c_char_p]
        lib.tfb_symm_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        lib.tfb_symm_close.argtypes = [C.c_void_p]
        lib.tfb_symm_free.argtypes = [C.c_void_p]
        # signalling state shared by the fused kernels of one stream: flags int32[world], epoch counter
        self.flags = self.alloc_bytes(4 * max(world, 32))
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.barrier()

    def alloc_bytes(self, nbytes: int) -> SymmBuffer:
        nbytes = (int(nbytes) + 511) // 512 * 512
        lib = _lib.lib()
        torch.cuda.set_device(self.device)
        p = C.c_void_p()
        h = C.create_string_buffer(64)
        _lib.check(lib.tfb_symm_alloc(nbytes, C.byref(p), h), "symm_alloc", 0)
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, bytes(h.raw), group=self.group)
        else:
            handles[0] = bytes(h.raw)
        ptrs = []
        for r, hb in enumerate(handles):
            if r == self.rank:
                ptrs.append(p.value)
            else:
                q = C.c_void_p()
                _lib.check(lib.tfb_symm_open(hb, C.byref(q)), "symm_open", 0)
                ptrs.append(q.value)
        buf = SymmBuffer(self, nbytes, p.value, ptrs)
        self.buffers.append(buf)
        return buf

    def alloc(self, numel: int, dtype) -> SymmBuffer:
        """Allocator hook used by FlatBuffers: returns a SymmBuffer holding ``numel`` elements."""
        return self.alloc_bytes(numel * torch.empty((), dtype=dtype).element_size())

    def barrier(self):
        """Device-side barrier on the current stream (bounded wait; see ops._lib.check_status)."""
        _lib.check(_lib.lib().tfb_comm_barrier(self.flags.ptrs.data_ptr(), self.epoch.data_ptr(), self.rank,
                                               self.world, _lib.status_word(self.device).data_ptr(), _lib.stream()),
                   "comm_barrier")

    def on_reset(self, fn):
        """Register a callable that puts a user's device-side bookkeeping (completion tickets, partial accumulators)
        back to its idle state; ``reset()`` runs all of them."""
        self._reset_hooks.append(fn)

    def reset(self):
        """Recovery after a bounded device wait ran out (``ops._lib.check_status`` raised ``KernelError``).

        A kernel that gives up returns before its last-CTA bookkeeping: completion tickets and accumulators keep partial
        counts and the ranks' epochs are out of step, so the next collective on this heap could see a stale "done" and
        overwrite buffers that are still in use.  Every rank of the group calls this (it is a host-side collective): the
        device is drained, the ranks agree on a fresh epoch above anything in flight, every local flag and the local
        epoch are set to it, the registered hooks clear tickets and accumulators, the status word is cleared, and one
        bounded device barrier proves that the flags work again."""
        torch.cuda.synchronize(self.device)
        e = self.epoch.clone().to(torch.int64)
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)
            dist.all_reduce(e, op=dist.ReduceOp.MAX, group=self.group)
        fresh = int(e.item()) + 1024
        self.flags.view(torch.int32).fill_(fresh)
        self.epoch.fill_(fresh)
        for fn in self._reset_hooks:
            fn()
        _lib.status_word(self.device).zero_()
        torch.cuda.synchronize(self.device)
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)
        self.barrier()
        torch.cuda.synchronize(self.device)
        _lib.check_status(self.device)

    def close(self):
        lib = _lib.lib()
        torch.cuda.synchronize(self.device)
        if dist.is_initialized():
            dist.barrier(group=self.group)
        for b in self.buffers:
            for r, q in enumerate(b.peer_ptrs):
                if r != self.rank:
                    lib.tfb_symm_close(q)
        if dist.is_initialized():
            dist.barrier(group=self.group)
        for b in self.buffers:
            lib.tfb_symm_free(b.local_ptr)
        self.buffers = []
