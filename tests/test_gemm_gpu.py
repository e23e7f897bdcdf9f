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
    assert err <= 1e-2 * ref.abs().max().item() + 1e-3, err


@pytest.mark.parametrize("M,N,K", [(640, 3504, 192), (1100, 7000, 128), (520, 3328, 64)])
def test_gemm_grouped_raster(M, N, K):
    """Wide outputs (more than twelve 256-column tiles, at least four row tiles) are walked in groups of eight tile columns:
    every output tile must still be produced exactly once, including the ragged last group."""
    for b_mn in (False, True):
        a, b = _mk(M, N, K, False, b_mn)
        c = F.gemm(a, b, b_mn=b_mn)
        torch.cuda.synchronize()
        _lib.check_status()
        ref = _ref(a, b, False, b_mn)
        err = (c.float() - ref).abs().max().item()
        assert err <= 1e-2 * ref.abs().max().item() + 1e-3, err


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


def _edge_values(tile, free):
    """Sizes around a tile edge: a dimension that is a row pitch of a TMA tensor map must stay a multiple of 8 elements
    (16 bytes), a free dimension may be any size."""
    return [1, tile - 1, tile, tile + 1] if free else [8, tile - 8, tile, tile + 8]


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_tile_edge_sweep(a_mn, b_mn):
    """M, N, K each at 1 (or 8), tile - 1, tile, tile + 1 (tile = 128 rows, 256 or 128 columns, 64 of K) in every operand
    layout, bf16 and fp32 outputs, within 1e-2 of the fp32 product's largest magnitude."""
    # which dimensions are contiguous (= row pitches): A [M,K] -> K; A stored [K,M] -> M; B [N,K] -> K; B stored [K,N] -> N;
    # C [M,N] -> N (an unaligned N takes the per-thread store path, which the free sizes of N exercise)
    m_free, k_free = not a_mn, a_mn and b_mn
    n_free = not b_mn
    worst = 0.0
    for M in _edge_values(128, m_free):
        for N in _edge_values(256, n_free) + ([128 + 8] if not n_free else [129]):
            for K in _edge_values(64, k_free) + [8 * 64 + 8]:
                a, b = _mk(M, N, K, a_mn, b_mn)
                ref = _ref(a, b, a_mn, b_mn)
                scale = ref.abs().max().item() + 1e-6
                c = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
                c32 = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
                e1 = (c.float() - ref).abs().max().item() / scale
                e2 = (c32 - ref).abs().max().item() / scale
                worst = max(worst, e1, e2)
                assert e1 <= 1e-2 and e2 <= 2e-3, (M, N, K, a_mn, b_mn, e1, e2)
    torch.cuda.synchronize()
    _lib.check_status()
    assert worst > 0.0
