"""Elementwise / normalisation / loss / optimiser kernels against the PyTorch fp32 statement of the
same op (the CPU branch of transformers_fusion_b200.ops.functional)."""
import pytest
import torch

from transformers_fusion_b200.ops import functional as F

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def close(a, b, tol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    assert (a - b).abs().max().item() <= tol * b.abs().max().item() + tol, (a - b).abs().max().item()


@pytest.mark.parametrize("H", [512, 768, 4096])
def test_rmsnorm_fwd_bwd(H):
    T = 300
    x = torch.randn(T, H, dtype=BF)
    r = torch.randn(T, H, dtype=BF)
    w = (1 + 0.1 * torch.randn(H)).to(BF)
    dy = torch.randn(T, H, dtype=BF)
    dres = torch.randn(T, H, dtype=BF)
    y0, h0, rstd0 = F.rmsnorm_fwd(x, w, 1e-5, r)
    dw0 = torch.zeros(H)
    dx0 = F.rmsnorm_bwd(dy, h0, w, rstd0, dw0, dres)
    y1, h1, rstd1 = F.rmsnorm_fwd(x.cuda(), w.cuda(), 1e-5, r.cuda())
    dw1 = torch.zeros(H, device="cuda")
    dx1 = F.rmsnorm_bwd(dy.cuda(), h1, w.cuda(), rstd1, dw1, dres.cuda())
    close(y1, y0); close(h1, h0); close(rstd1, rstd0, 1e-3); close(dx1, dx0); close(dw1, dw0)


def test_layernorm_fwd_bwd():
    T, H = 200, 768
    x = torch.randn(T, H, dtype=BF) + 0.5
    w = (1 + 0.1 * torch.randn(H)).to(BF)
    b = (0.1 * torch.randn(H)).to(BF)
    dy = torch.randn(T, H, dtype=BF)
    y0, h0, rstd0, mean0 = F.layernorm_fwd(x, w, b, 1e-5)
    dw0, db0 = torch.zeros(H), torch.zeros(H)
    dx0 = F.layernorm_bwd(dy, h0, w, rstd0, mean0, dw0, db0)
    y1, h1, rstd1, mean1 = F.layernorm_fwd(x.cuda(), w.cuda(), b.cuda(), 1e-5)
    dw1, db1 = torch.zeros(H, device="cuda"), torch.zeros(H, device="cuda")
    dx1 = F.layernorm_bwd(dy.cuda(), h1, w.cuda(), rstd1, mean1, dw1, db1)
    close(y1, y0); close(dx1, dx0); close(dw1, dw0); close(db1, db0)


def test_rope_roundtrip_and_ref():
    T, S, nh, D = 256, 128, 10, 64
    ld = 12 * D
    x = torch.randn(T, ld, dtype=BF)
    cos, sin = F.rope_tables(D, 512, 10000.0)
    ref = F.rope_(x.clone(), cos, sin, nh, D, S)
    g = x.clone().cuda()
    F.rope_(g, cos.cuda(), sin.cuda(), nh, D, S)
    close(g, ref)
    F.rope_(g, cos.cuda(), sin.cuda(), nh, D, S, backward=True)
    close(g, x, 3e-2)


@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_glu(act):
    M, Fh = 333, 1408
    x = torch.randn(M, 2 * Fh, dtype=BF)
    d = torch.randn(M, Fh, dtype=BF)
    close(F.glu_fwd(x.cuda(), act), F.glu_fwd(x, act))
    close(F.glu_bwd(x.cuda(), d.cuda(), act), F.glu_bwd(x, d, act))
    # device-side row count: only the first rows are computed, the rest of the output is left alone
    rows = torch.tensor([200], dtype=torch.int32, device="cuda")
    close(F.glu_fwd(x.cuda(), act, rows=rows)[:200], F.glu_fwd(x, act)[:200])
    close(F.glu_bwd(x.cuda(), d.cuda(), act, rows=rows)[:200], F.glu_bwd(x, d, act)[:200])


def test_embedding():
    V, H, T, S = 1000, 512, 640, 64
    W = torch.randn(V, H, dtype=BF)
    P = torch.randn(S, H, dtype=BF)
    ids = torch.randint(0, V, (T,))
    close(F.embedding_fwd(ids.cuda(), W.cuda(), P.cuda(), S), F.embedding_fwd(ids, W, P, S))
    d = torch.randn(T, H, dtype=BF)
    dW0, dP0 = torch.zeros(V, H), torch.zeros(S, H)
    F.embedding_bwd(ids, d, dW0, dP0, S)
    dW1, dP1 = torch.zeros(V, H, device="cuda"), torch.zeros(S, H, device="cuda")
    F.embedding_bwd(ids.cuda(), d.cuda(), dW1, dP1, S)
    close(dW1, dW0); close(dP1, dP0)


@pytest.mark.parametrize("V,ls,zw", [(32000, 0.0, 0.0), (32000, 0.1, 1e-3), (1003, 0.1, 1e-3)])
def test_cross_entropy(V, ls, zw):
    T = 97
    z = (3 * torch.randn(T, V)).to(BF)
    lab = torch.randint(0, V, (T,))
    lab[5] = -100
    sc = torch.tensor([1.0 / 96])
    z0 = z.clone()
    l0 = F.cross_entropy_fwd_bwd(z0, lab, sc, label_smoothing=ls, z_weight=zw)
    z1 = z.clone().cuda()
    l1 = F.cross_entropy_fwd_bwd(z1, lab.cuda(), sc.cuda(), label_smoothing=ls, z_weight=zw)
    close(l1, l0, 1e-2)
    assert (z1.float().cpu() - z0.float()).abs().max().item() < 2e-4


def test_adamw_and_clip():
    n = 100003
    p, g = torch.randn(n), torch.randn(n)
    m, v = torch.zeros(n), torch.zeros(n)
    plp = torch.zeros(n, dtype=BF)
    P, G, M, V, PL = p.cuda(), g.cuda(), m.cuda(), v.cuda(), plp.cuda()
    ss0, ss1 = torch.zeros(()), torch.zeros((), device="cuda")
    F.sumsq(g, ss0); F.sumsq(G, ss1)
    close(ss1, ss0, 1e-4)
    n0, c0, n1, c1 = torch.zeros(()), torch.zeros(()), torch.zeros((), device="cuda"), torch.zeros((), device="cuda")
    F.clip_factor(ss0, 1.0, 1.0, n0, c0); F.clip_factor(ss1, 1.0, 1.0, n1, c1)
    close(c1, c0, 1e-4)
    for step in (1, 2):
        g2, G2 = g.clone(), G.clone()
        F.adamw_(p, g2, m, v, plp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, c0)
        F.adamw_(P, G2, M, V, PL, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, c1)
        assert G2.abs().max().item() == 0
    close(P, p, 1e-4); close(M, m, 1e-4); close(V, v, 1e-4); close(PL, plp, 1e-2)


@pytest.mark.gpu
def test_bounds_check_build_reports_first_bad_index():
    """The -DTFB_BOUNDS_CHECK library records an out-of-range token id and label (the accesses themselves stay clamped /
    skipped, so nothing faults); the release library ignores them silently.  Runs in a child process because the library
    variant is chosen at load time."""
    import os
    import subprocess
    import sys
    code = r'''
import torch
from transformers_fusion_b200.ops import _lib, functional as F
assert _lib.lib_path().name == "libtfb_kernels_check.so"
W = torch.randn(32, 64, device="cuda").bfloat16()
ids = torch.tensor([1, 2, 99, 3], device="cuda")
out = F.embedding_fwd(ids, W, None, 0)
logits = torch.randn(4, 32, device="cuda").bfloat16()
labels = torch.tensor([1, -100, 77, 5], device="cuda")
F.cross_entropy_fwd_bwd(logits, labels, want_grad=False)
torch.cuda.synchronize()
rep = _lib.bounds_report()
assert rep["elementwise"][0] >= 1 and rep["elementwise"][1:] == (1, 99, 32), rep   # one hit per 8-column chunk of the row
assert rep["loss_optim"][0] == 1 and rep["loss_optim"][1:] == (3, 77, 32), rep
assert _lib.bounds_report()["elementwise"][0] == 0
assert torch.equal(out[2], W[0])
# paged KV cache: a slot beyond the pool is skipped, a block-table page beyond the pool reads page 0
from transformers_fusion_b200.inference.kv_cache import PAGE, PagedKVCache
cache = PagedKVCache(1, 4, 2, 64, "bf16", "cuda")
src = torch.randn(3, 2 * 2 * 64, device="cuda").bfloat16()
cache.append(0, src, 0, 128, torch.tensor([0, 1, 4 * PAGE + 5], device="cuda"))
q = torch.randn(1, 4 * 64, device="cuda").bfloat16()
bt = torch.tensor([[0, 9]], dtype=torch.int32, device="cuda")
o = cache.decode(0, q, bt, torch.tensor([PAGE + 2], dtype=torch.int32, device="cuda"), 4)
torch.cuda.synchronize()
rep = _lib.bounds_report()["paged_attention"]
assert rep[0] >= 2 and rep[1] in (51, 52) and rep[3] in (4 * PAGE, 4), rep
assert torch.isfinite(o.float()).all()
print("ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, cwd=root,
                       env=dict(os.environ, TFB_BOUNDS_CHECK="1"))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
