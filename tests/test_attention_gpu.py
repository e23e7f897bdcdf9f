"""tcgen05 flash attention against an fp32 PyTorch reference (causal / full, GQA, ragged lengths)."""
import math

import pytest
import torch

from transformers_fusion_b200.ops import _lib, functional as F

pytestmark = pytest.mark.gpu


def _qkv(B, S, Hq, Hkv, D):
    ld = (Hq + 2 * Hkv) * D
    return torch.randn(B * S, ld, device="cuda", dtype=torch.bfloat16)


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [
    (1, 128, 1, 1, 64, True), (2, 256, 4, 2, 64, True), (1, 1024, 8, 8, 64, True), (2, 200, 4, 1, 64, True),
    (1, 384, 2, 2, 64, False), (1, 300, 2, 1, 64, False), (1, 512, 4, 2, 128, True), (2, 130, 2, 2, 128, False),
])
def test_attn_fwd(B, S, Hq, Hkv, D, causal):
    qkv = _qkv(B, S, Hq, Hkv, D)
    kc, vc = Hq * D, (Hq + Hkv) * D
    o, lse = F.attn_fwd(qkv, qkv, qkv, B, S, Hq, Hkv, D, causal=causal, k_col0=kc, v_col0=vc)
    torch.cuda.synchronize()
    _lib.check_status()
    ro, rlse, _ = F.attn_ref(qkv, qkv, qkv, B, S, Hq, Hkv, D, 1 / math.sqrt(D), causal, 0, kc, vc)
    assert (o.float() - ro).abs().max().item() < 3e-2
    assert (lse - rlse).abs().max().item() < 2e-2


@pytest.mark.parametrize("B,S,Skv,Hq,Hkv,D,causal", [
    (1, 128, 256, 2, 1, 64, True), (1, 37, 300, 4, 2, 64, True), (2, 200, 456, 4, 4, 128, True), (1, 1, 129, 2, 2, 64, True),
    (1, 260, 261, 2, 1, 128, True), (1, 100, 356, 2, 2, 64, False), (1, 513, 1200, 8, 2, 128, True),
])
def test_attn_fwd_longer_keys(B, S, Skv, Hq, Hkv, D, causal):
    """The S queries are the last S positions of a sequence of Skv keys (a prompt suffix behind a cached prefix): query i
    sees keys 0 .. i + Skv - S."""
    q = torch.randn(B * S, Hq * D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B * Skv, Hkv * D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B * Skv, Hkv * D, device="cuda", dtype=torch.bfloat16)
    o, lse = F.attn_fwd(q, k, v, B, S, Hq, Hkv, D, causal=causal, kv_len=Skv)
    torch.cuda.synchronize()
    _lib.check_status()
    ro, rlse, _ = F.attn_ref(q, k, v, B, S, Hq, Hkv, D, 1 / math.sqrt(D), causal, kv_len=Skv)
    assert (o.float() - ro).abs().max().item() < 3e-2
    assert (lse - rlse).abs().max().item() < 2e-2


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [
    (1, 128, 1, 1, 64, True), (2, 256, 4, 2, 64, True), (1, 1024, 8, 8, 64, True), (2, 200, 4, 1, 64, True),
    (1, 300, 2, 1, 64, False), (1, 512, 4, 2, 128, True), (2, 130, 2, 2, 128, False),
])
def test_attn_bwd(B, S, Hq, Hkv, D, causal):
    qkv = _qkv(B, S, Hq, Hkv, D)
    kc, vc = Hq * D, (Hq + Hkv) * D
    dout = torch.randn(B * S, Hq * D, device="cuda", dtype=torch.bfloat16)
    o, lse = F.attn_fwd(qkv, qkv, qkv, B, S, Hq, Hkv, D, causal=causal, k_col0=kc, v_col0=vc)
    dqkv = torch.full_like(qkv, float("nan"))
    F.attn_bwd(qkv, qkv, qkv, o, dout, lse, dqkv, B, S, Hq, Hkv, D, causal=causal, k_col0=kc, v_col0=vc)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = torch.zeros_like(qkv).cpu()
    c = qkv.cpu()
    F.attn_bwd(c, c, c, None, dout.cpu(), None, ref, B, S, Hq, Hkv, D, causal=causal, k_col0=kc, v_col0=vc)
    err = (dqkv.float().cpu() - ref.float()).abs()
    scale = ref.float().abs().max().item()
    assert torch.isfinite(dqkv.float()).all()
    assert err.max().item() < 3e-2 * scale + 2e-2, (err.max().item(), scale)
