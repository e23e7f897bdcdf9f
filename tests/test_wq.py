"""Fused-dequant GEMM: packing round trip on CPU, kernel against the fp32 product of the dequantised weights on GPU."""
import pytest
import torch

from transformers_fusion_b200.quant import wq


@pytest.mark.parametrize("fmt,group,tol", [("int8", 64, 0.012), ("int4", 32, 0.16), ("mxfp8", 32, 0.07), ("fp4", 32, 0.3), ("ternary", 32, 1.2)])
def test_pack_roundtrip(fmt, group, tol):
    torch.manual_seed(0)
    w = torch.randn(200, 150)
    pw = wq.pack_weight(w, fmt, group)
    assert pw.Np == 256 and pw.Kp == 192 and pw.codes.dtype == torch.uint8
    d = wq.dequant(pw)
    assert d.shape == w.shape
    rel = float((d - w).abs().max() / w.abs().max())
    assert rel < tol, rel
    assert pw.codes.numel() == 256 * 192 * wq.BITS[pw.fmt] // 8
    if fmt == "mxfp8":
        s = pw.scales.float()
        assert torch.equal(torch.exp2(torch.round(torch.log2(s))), s)       # E8M0-representable
    x = torch.randn(5, 150)
    assert torch.allclose(wq.gemm_wq(x, pw), x @ d.t(), atol=1e-4)


def test_device_format_choice():
    assert wq.device_format_for("Q_8") == ("int8", 64) and wq.device_format_for("Q_G_4") == ("int4", 32)
    assert wq.device_format_for("Q_4_K_M")[0] == "fp4" and wq.device_format_for("Q_2")[0] == "ternary"
    assert wq.device_format_for("Q_16") == (None, 0) and wq.device_format_for("Q_MX_8_5")[0] == "mxfp8"


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,group", [("int8", 64), ("int8", 32), ("int4", 32), ("mxfp8", 32), ("fp4", 64), ("ternary", 32)])
@pytest.mark.parametrize("M", [1, 8, 16, 17, 200, 2176])
def test_gemm_wq_gpu(fmt, group, M):
    torch.manual_seed(1)
    N, K = 384, 1024
    w = torch.randn(N, K) * 0.05
    pw = wq.pack_weight(w.cuda(), fmt, group)
    x = torch.randn(M, K).bfloat16().cuda()
    bias = torch.randn(N).bfloat16().cuda()
    ref = x.float() @ wq.dequant(pw).t() + bias.float()
    for splits in (0, 1):
        y = wq.gemm_wq(x, pw, bias, splits=splits)
        err = (y.float() - ref).abs().max() / ref.abs().max()
        assert err < 1.5e-2, (fmt, M, splits, float(err))
    from transformers_fusion_b200.ops import _lib
    torch.cuda.synchronize()
    assert int(_lib.status_word(x.device)[0]) == 0


@pytest.mark.gpu
def test_quant_linear_module():
    torch.manual_seed(2)
    lin = wq.QuantLinear(torch.randn(256, 512).cuda() * 0.1, "int4", 32)
    x = torch.randn(2, 3, 512).bfloat16().cuda()
    y = lin(x)
    assert y.shape == (2, 3, 256) and "bits/weight" in repr(lin)
    ref = x.float().view(-1, 512) @ wq.dequant(lin.pw).t()
    assert (y.float().view(-1, 256) - ref).abs().max() / ref.abs().max() < 1.5e-2


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,group", [("int8", 64), ("int4", 32), ("mxfp8", 32), ("fp4", 32), ("ternary", 64)])
def test_dequant_bf16_image_is_exact(fmt, group):
    """The device image equals the fp32 oracle rounded to bf16, bit for bit."""
    torch.manual_seed(3)
    pw = wq.pack_weight(torch.randn(256, 320).cuda() * 0.07, fmt, group)
    img = wq.dequant_bf16(pw)
    ref = torch.zeros(pw.Np, pw.Kp, device="cuda")
    ref[: pw.N, : pw.K] = wq.dequant(pw)
    assert torch.equal(img.float(), ref.bfloat16().float())
