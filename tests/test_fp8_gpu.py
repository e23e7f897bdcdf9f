"""Block-scaled FP8 quantisers and tcgen05 GEMM against the PyTorch fp32 statement."""
import pytest
import torch

from transformers_fusion_b200.ops import _lib
from transformers_fusion_b200.quant import fp8

pytestmark = pytest.mark.gpu


def test_quantisers_match_reference():
    x = torch.randn(300, 640, dtype=torch.bfloat16) * 3
    w = torch.randn(260, 640, dtype=torch.bfloat16)
    q0, s0 = fp8.quant_act_1x128(x)
    q1, s1 = fp8.quant_act_1x128(x.cuda())
    assert torch.allclose(s0, s1.cpu(), rtol=1e-6)
    assert (fp8.dequant(q0, s0, 1) - fp8.dequant(q1.cpu(), s1.cpu(), 1)).abs().max() <= 33 * s0.max()  # at most one e4m3 step in the top binade
    assert (q0 != q1.cpu()).float().mean() < 1e-3
    qw0, sw0 = fp8.quant_weight_128x128(w)
    qw1, sw1 = fp8.quant_weight_128x128(w.cuda())
    assert torch.allclose(sw0, sw1.cpu(), rtol=1e-6)
    assert (qw0 != qw1.cpu()).float().mean() < 1e-3


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1000, 520, 1152), (4096, 4096, 2048)])
def test_gemm_fp8_dense(M, N, K):
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    qa, sa = fp8.quant_act_1x128(x)
    qb, sb = fp8.quant_weight_128x128(w)
    c = fp8.gemm_fp8(qa, sa, qb, sb)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = fp8.dequant(qa, sa, 1) @ fp8.dequant(qb, sb, 128).t()
    assert (c.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    # and the quantised product is close to the bf16 product
    full = x.float() @ w.float().t()
    assert (c.float() - full).norm().item() / full.norm().item() < 0.08


def test_gemm_fp8_grouped():
    E, N, K = 4, 256, 512
    tiles = [0, 0, 2, -1, 3, 1, 1]
    M = 128 * len(tiles)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16)
    qa, sa = fp8.quant_act_1x128(x)
    qb, sb = fp8.quant_weight_128x128(w)
    eo = torch.tensor(tiles, dtype=torch.int32, device="cuda")
    c = fp8.gemm_fp8(qa, sa, qb, sb, eo)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = fp8.gemm_fp8(qa.cpu(), sa.cpu(), qb.cpu(), sb.cpu(), eo.cpu())
    assert (c.float().cpu() - ref.float()).abs().max().item() <= 1e-2 * ref.float().abs().max().item() + 1e-2
