"""tcgen05 bf16 GEMM against a PyTorch fp32 reference: every operand layout, ragged tile edges,
epilogues, fp32 output and split-K accumulation."""
import pytest
import torch

from transformers_fusion_b200.ops import _lib, functional as F

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = (a.t() if a_mn else a).float()
    B = (b if b_mn else b.t()).float()
    return A @ B


def _mk(M, N, K, a_mn, b_mn):
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    return a, b


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (384, 128, 192), (1000, 776, 328), (72, 40, 1096)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    a, b = _mk(M, N, K, a_mn, b_mn)
    c = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = _ref(a, b, a_mn, b_mn)
    err = (c.float() - ref).abs().max().item()
    assert err <= 0.02 * ref.abs().max().item() + 1e-2, err


def test_gemm_epilogue():
    M, N, K = 512, 768, 256
    a, b = _mk(M, N, K, False, False)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    for act in (None, "relu", "gelu", "silu"):
        c = F.gemm(a, b, bias=bias, residual=res, act=act, alpha=0.5)
        ref = F._act_ref(0.5 * _ref(a, b, False, False) + bias.float(), act) + res.float()
        torch.cuda.synchronize()
        _lib.check_status()
        assert (c.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-2


def test_gemm_fp32_and_splitk_accumulate():
    # weight-gradient shape: small output, long reduction -> split-K with fp32 atomics
    M, N, K = 512, 512, 16384
    a, b = _mk(M, N, K, True, True)
    out = torch.ones(M, N, device="cuda", dtype=torch.float32)
    F.gemm(a, b, a_mn=True, b_mn=True, out=out, accumulate=True)
    ref = _ref(a, b, True, True) + 1.0
    torch.cuda.synchronize()
    _lib.check_status()
    assert (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-2
    c = F.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    assert (c - (ref - 1.0)).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-2


def test_gemm_many_tiles_persistent():
    M, N, K = 4096, 4096, 1024
    a, b = _mk(M, N, K, False, False)
    c = F.gemm(a, b)
    ref = _ref(a, b, False, False)
    torch.cuda.synchronize()
    _lib.check_status()
    assert (c.float() - ref).abs().max().item() <= 0.02 * ref.abs().max().item() + 1e-2
