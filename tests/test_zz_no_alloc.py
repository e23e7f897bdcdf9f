"""The allocation-free attention-backward entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory where they call it (inside a stream capture,
under a fixed memory budget, or where cudaMalloc's device-wide synchronisation is unacceptable), so
``tfb_attn_bwd_noalloc`` keeps its scratch in a fixed array inside the library.  Its gradients must
equal those of the ordinary entry point, call after call, because every call reuses the same array."""
import ctypes as C
import math

import pytest
import torch

from transformers_fusion_b200.ops import _lib, functional as F

pytestmark = pytest.mark.gpu

c_p, c_ll, c_i, c_f = C.c_void_p, C.c_longlong, C.c_int, C.c_float
SIG = [c_p, c_ll, c_i, c_p, c_ll, c_i, c_p, c_ll, c_i, c_p, c_ll, c_p, c_ll, c_p,
       c_p, c_ll, c_i, c_p, c_ll, c_i, c_p, c_ll, c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_i, c_p, c_p]


def _call(fn, qkv, o, dout, lse, dqkv, B, S, Hq, Hkv, D):
    kc, vc = Hq * D, (Hq + Hkv) * D
    p, ld = qkv.data_ptr(), qkv.stride(0)
    dp, ldd = dqkv.data_ptr(), dqkv.stride(0)
    return fn(p, ld, 0, p, ld, kc, p, ld, vc, o.data_ptr(), o.stride(0), dout.data_ptr(), dout.stride(0),
              lse.data_ptr(), dp, ldd, 0, dp, ldd, kc, dp, ldd, vc, B, S, Hq, Hkv, D, 1.0 / math.sqrt(D), 1,
              _lib.status_word(qkv.device).data_ptr(), torch.cuda.current_stream().cuda_stream)


def _fp32_statement(qkv, dout, B, S, Hq, Hkv, D):
    """Gradients of causal grouped-query attention by torch autograd in fp32 on the same bf16 inputs."""
    x = qkv.float().detach().requires_grad_(True)
    q = x[:, :Hq * D].view(B, S, Hq, D).transpose(1, 2)
    k = x[:, Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
    v = x[:, (Hq + Hkv) * D:].view(B, S, Hkv, D).transpose(1, 2).repeat_interleave(Hq // Hkv, 1)
    s = (q @ k.transpose(-1, -2)) / math.sqrt(D)
    s = s.masked_fill(torch.ones(S, S, device=x.device, dtype=torch.bool).triu(1), float("-inf"))
    o = (s.softmax(-1) @ v).transpose(1, 2).reshape(B * S, Hq * D)
    o.backward(dout.float())
    return x.grad


def test_noalloc_matches_regular_entry_point_twice():
    """Compared with the ordinary entry point on both calls (that one is checked against fp32 in
    test_attention_gpu.py) and, on the first call, directly with the fp32 statement as well."""
    lib = _lib.lib()
    fn = lib.tfb_attn_bwd_noalloc
    fn.argtypes, fn.restype = SIG, c_i
    for n, (B, S, Hq, Hkv, D) in enumerate([(2, 384, 4, 2, 64), (1, 200, 2, 1, 128)]):   # two calls in a row
        qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
        dout = torch.randn(B * S, Hq * D, device="cuda", dtype=torch.bfloat16)
        kc, vc = Hq * D, (Hq + Hkv) * D
        o, lse = F.attn_fwd(qkv, qkv, qkv, B, S, Hq, Hkv, D, k_col0=kc, v_col0=vc)
        ref = torch.zeros_like(qkv)
        F.attn_bwd(qkv, qkv, qkv, o, dout, lse, ref, B, S, Hq, Hkv, D, k_col0=kc, v_col0=vc)
        got = torch.full_like(qkv, float("nan"))
        free_before = torch.cuda.mem_get_info()[0]
        assert _call(fn, qkv, o, dout, lse, got, B, S, Hq, Hkv, D) == 0
        torch.cuda.synchronize()
        _lib.check_status()
        if n > 0:   # past the first call (module load, address look-up) a call leaves device memory untouched
            assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20)
        scale = ref.float().abs().max().item()
        assert torch.isfinite(got.float()).all()
        assert (got.float() - ref.float()).abs().max().item() < 3e-2 * scale + 2e-2
        if n == 0:
            exact = _fp32_statement(qkv, dout, B, S, Hq, Hkv, D)
            assert (got.float() - exact).abs().max().item() < 3e-2 * exact.abs().max().item() + 2e-2


def test_noalloc_rejects_oversize():
    lib = _lib.lib()
    fn = lib.tfb_attn_bwd_noalloc
    fn.argtypes, fn.restype = SIG, c_i
    t = torch.zeros(16, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(16, device="cuda", dtype=torch.float32)
    # 8 Mi rows > 4 Mi limit: must be refused before anything is launched or dereferenced
    rc = fn(t.data_ptr(), 64, 0, t.data_ptr(), 64, 0, t.data_ptr(), 64, 0, t.data_ptr(), 64, t.data_ptr(), 64,
            f.data_ptr(), t.data_ptr(), 64, 0, t.data_ptr(), 64, 0, t.data_ptr(), 64, 0, 8, 1024 * 1024, 1, 1, 64, 0.125,
            1, None, None)
    assert rc == -3
