"""ZeRO-1/2 gradient and parameter path on the fused peer-memory kernels.

The flat fp32 gradient buffer and the flat bf16 parameter buffer live in symmetric memory.  One
optimizer step is three launches on the training stream, with no NCCL call and no host sync:

  1. ``tfb_zero_reduce_scatter``  — flag barrier ("backward finished everywhere"), peer loads of the W
     copies of this rank's shard, 1/W scale, squared norm of the reduced shard, partial norm pushed
     to every peer;
  2. ``tfb_zero_adamw_allgather`` — global norm from the W partials, clip, AdamW on the fp32 master
     shard, refreshed bf16 parameters stored into every rank's buffer, gradients cleared;
  3. ``tfb_zero_wait``            — parameters from every peer have landed.

Reference counterparts: ZeroOptimizer::reduce_scatter_grads / step / all_gather_params
(src/trainer/zero_optimizer_core.cpp:173-298), DDP bucket all-reduce (src/trainer/ddp.cpp:113-173).
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _lib


class _Desc(C.Structure):
    _fields_ = [("flag_ptrs", C.c_void_p), ("epoch", C.c_void_p), ("rank", C.c_int), ("world", C.c_int),
                ("status", C.c_void_p), ("grad_ptrs", C.c_void_p), ("param_ptrs", C.c_void_p),
                ("norm_ptrs", C.c_void_p), ("numel", C.c_longlong), ("master", C.c_void_p), ("m", C.c_void_p),
                ("v", C.c_void_p), ("hyper", C.c_void_p), ("beta1", C.c_float), ("beta2", C.c_float),
                ("eps", C.c_float), ("wd", C.c_float), ("max_norm", C.c_float), ("accum", C.c_void_p),
                ("ticket", C.c_void_p), ("grad_norm_out", C.c_void_p)]


class FusedZero:
    def __init__(self, flat, opt, symm, rank, world, max_ctas=0):
        assert flat.symm_params is not None and flat.symm_grads is not None, \
            "FusedZero needs flat buffers allocated from the symmetric heap"
        assert flat.numel % (8 * world) == 0
        self.flat, self.opt, self.symm, self.rank, self.world, self.max_ctas = flat, opt, symm, rank, world, max_ctas
        dev = flat.params.device
        self.norm_slots = symm.alloc_bytes(4 * max(world, 32))
        self.accum = torch.zeros(4, dtype=torch.float32, device=dev)
        self.ticket = torch.zeros(4, dtype=torch.int32, device=dev)
        symm.on_reset(lambda: (self.accum.zero_(), self.ticket.zero_()))
        lib = _lib.lib()
        for name in ("tfb_zero_reduce_scatter", "tfb_zero_adamw_allgather"):
            fn = getattr(lib, name)
            fn.argtypes = [C.POINTER(_Desc), C.c_int, C.c_void_p]
            fn.restype = C.c_int
        lib.tfb_zero_wait.argtypes = [C.POINTER(_Desc), C.c_void_p]
        lib.tfb_zero_wait.restype = C.c_int
        d = _Desc()
        d.flag_ptrs, d.epoch = symm.flags.ptrs.data_ptr(), symm.epoch.data_ptr()
        d.rank, d.world = rank, world
        d.status = _lib.status_word(dev).data_ptr()
        d.grad_ptrs, d.param_ptrs = flat.symm_grads.ptrs.data_ptr(), flat.symm_params.ptrs.data_ptr()
        d.norm_ptrs = self.norm_slots.ptrs.data_ptr()
        d.numel = flat.numel
        d.master, d.m, d.v = opt.master.data_ptr(), opt.m.data_ptr(), opt.v.data_ptr()
        d.hyper = opt.hyper.data_ptr()
        d.beta1, d.beta2, d.eps, d.wd = opt.betas[0], opt.betas[1], opt.eps, opt.weight_decay
        d.max_norm = opt.max_grad_norm
        d.accum, d.ticket = self.accum.data_ptr(), self.ticket.data_ptr()
        d.grad_norm_out = opt.grad_norm.data_ptr()
        self.desc = d

    def step(self):
        """Hyper-parameters of this step must already be staged (FlatAdamW.stage_hyper)."""
        lib, s = _lib.lib(), _lib.stream()
        _lib.check(lib.tfb_zero_reduce_scatter(C.byref(self.desc), self.max_ctas, s), "zero_reduce_scatter")
        _lib.check(lib.tfb_zero_adamw_allgather(C.byref(self.desc), self.max_ctas, s), "zero_adamw_allgather")
        _lib.check(lib.tfb_zero_wait(C.byref(self.desc), s), "zero_wait")
