"""ctypes binding to ``lib/libtfb_kernels.so`` (the sm_100a kernels).

The library exposes a plain C ABI: every entry point takes raw device pointers, sizes and the CUDA
stream handle, and returns 0 on success.  Python passes ``tensor.data_ptr()`` and the current torch
stream, so launches are ordered with the surrounding PyTorch work and can be captured in CUDA
graphs.  On a machine with a GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_lib = None
_status = {}

c_p = C.c_void_p
c_i = C.c_int
c_ll = C.c_longlong
c_f = C.c_float

_SIGS = {
    "tfb_sm_count": [],
    "tfb_gemm_bf16": [c_p, c_ll, c_i, c_p, c_ll, c_i, c_p, c_ll, c_i, c_i, c_i, c_p, c_p, c_ll, c_f, c_i, c_i, c_i, c_p, c_p],
    "tfb_rmsnorm_fwd": [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_f, c_p],
    "tfb_rmsnorm_bwd": [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_p],
    "tfb_layernorm_fwd": [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_f, c_p],
    "tfb_layernorm_bwd": [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_p],
    "tfb_rope": [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_ll, c_i, c_p],
    "tfb_glu_fwd": [c_p, c_p, c_ll, c_i, c_i, c_p],
    "tfb_glu_bwd": [c_p, c_p, c_p, c_ll, c_i, c_i, c_p],
    "tfb_glu_fwd_rows": [c_p, c_p, c_ll, c_i, c_i, c_p, c_p],
    "tfb_glu_bwd_rows": [c_p, c_p, c_p, c_ll, c_i, c_i, c_p, c_p],
    "tfb_act_fwd": [c_p, c_p, c_ll, c_i, c_p],
    "tfb_act_bwd": [c_p, c_p, c_p, c_ll, c_i, c_p],
    "tfb_embedding_fwd": [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p],
    "tfb_embedding_bwd": [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p],
    "tfb_add_bf16": [c_p, c_p, c_p, c_ll, c_p],
    "tfb_cross_entropy": [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_ll, c_ll, c_f, c_f, c_p],
    "tfb_sumsq_f32": [c_p, c_ll, c_p, c_p],
    "tfb_clip_factor": [c_p, c_f, c_f, c_p, c_p, c_p, c_p],
    "tfb_adamw": [c_p, c_p, c_p, c_p, c_p, c_ll, c_f, c_f, c_f, c_f, c_f, c_i, c_p, c_i, c_p, c_p],
    "tfb_lion_sgd": [c_p, c_p, c_p, c_p, c_ll, c_f, c_f, c_f, c_f, c_i, c_p, c_i, c_p],
    "tfb_cast_f32_bf16": [c_p, c_p, c_ll, c_p],
    "tfb_cast_bf16_f32": [c_p, c_p, c_ll, c_p],
}


class KernelError(RuntimeError):
    pass


def bounds_check_build() -> bool:
    return os.environ.get("TFB_BOUNDS_CHECK", "") not in ("", "0")


def lib_path() -> Path:
    return _LIB_DIR / ("libtfb_kernels_check.so" if bounds_check_build() else "libtfb_kernels.so")


def bounds_report(reset: bool = True) -> dict:
    """Bounds-check build only: {unit: (count, site, index, limit)} of the first out-of-range index each unit saw
    (sites: 1 embedding id, 2 embedding-gradient id, 3 cross-entropy label, 5 routed expert id, 11 gather block of a
    fused GEMM, 12 expert of a grouped-GEMM row tile, 21 row owner of the sharded embedding, 31 vocabulary-parallel label,
    41 destination row of an expert-parallel dispatch, 51 KV-cache slot of an append, 52 page of a paged-decode block
    table, 53 page of a KV gather)."""
    out = {}
    if not bounds_check_build():
        return out
    for unit in ("elementwise", "loss_optim", "moe_routing", "gemm_bf16", "fsdp_fused", "loss_vocab_parallel", "ep_fused",
                 "paged_attention"):
        fn = getattr(lib(), f"tfb_bounds_report_{unit}", None)
        if fn is None:
            continue
        fn.argtypes, fn.restype = [c_p, c_i], c_i
        buf = (C.c_ulonglong * 4)()
        check(fn(C.addressof(buf), int(reset)), f"bounds_report_{unit}")
        idx = buf[2] - (1 << 64) if buf[2] >= (1 << 63) else buf[2]
        out[unit] = (int(buf[0]), int(buf[1]), int(idx), int(buf[3]))
    return out


def available() -> bool:
    return lib_path().exists()


def lib():
    """Load (once) and return the kernel library; build it first if the shared object is absent."""
    global _lib
    if _lib is not None:
        return _lib
    p = lib_path()
    if not p.exists():
        if os.environ.get("TFB_NO_AUTOBUILD"):
            raise KernelError(f"{p} is missing; run `python -m transformers_fusion_b200.build`")
        from .. import build as _build
        _build.build_kernels(bounds_check=bounds_check_build())
    _lib = C.CDLL(str(p))
    for name, sig in _SIGS.items():
        try:
            fn = getattr(_lib, name)
        except AttributeError:
            continue
        fn.argtypes = sig
        fn.restype = c_i
    return _lib


def register(name: str, sig):
    """Declare the signature of an entry point defined by another module (attention, comm, quant)."""
    _SIGS[name] = sig
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = sig
        fn.restype = c_i


LAUNCHES = [0]  # kernels launched through this binding (graph replays are counted by the engine)


def check(rc: int, what: str, n: int = 1):
    LAUNCHES[0] += n
    if rc != 0:
        if rc > 0:
            raise KernelError(f"{what}: CUDA error {rc} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no gpu'})")
        raise KernelError(f"{what}: tfb error {rc} (-1 bad shape/alignment, -2 driver entry point, -3 size limit)")


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write a code into when a wait runs out."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(8, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = t
    return t


_STATUS_NAMES = {
    1: "operand stage never arrived (TMA)", 2: "stage never released (MMA)", 3: "accumulator never committed",
    4: "accumulator never drained", 5: "copies still in flight at exit", 6: "peer flag never set", 7: "bad argument",
}


def check_status(device=None, reset=True):
    """Synchronising read of the status word; raises if any kernel reported a wait that ran out."""
    t = status_word(device)
    code = int(t[0].item())
    if code:
        if reset:
            t.zero_()
        raise KernelError(f"device status {code}: {_STATUS_NAMES.get(code, 'unknown')}")
