"""Paged KV cache (bf16 / fp8 / 4-bit) append + decode attention, and the sampling kernel, against
their host statements."""
import math

import pytest
import torch

from transformers_fusion_b200.inference.kv_cache import PAGE, PagedKVCache
from transformers_fusion_b200.inference import sampler as S
from transformers_fusion_b200.ops import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["bf16", "fp8", "q4"])
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 64), (4, 1, 128), (4, 4, 64), (8, 1, 128), (4, 2, 64)])
def test_paged_append_and_decode(mode, Hq, Hkv, D):
    B, pages = 6, 112
    lens = torch.tensor([1, 17, 100, 255, 33, 700], dtype=torch.int32)
    ld = (Hq + 2 * Hkv) * D
    caches = {d: PagedKVCache(1, pages, Hkv, D, mode, d) for d in ("cpu", "cuda")}
    max_pages = (int(lens.max()) + PAGE - 1) // PAGE
    bt = torch.zeros(B, max_pages, dtype=torch.int32)
    perm = torch.randperm(pages)
    nxt = 0
    srcs, slots = [], []
    for b in range(B):
        n = int(lens[b])
        for i in range((n + PAGE - 1) // PAGE):
            bt[b, i] = perm[nxt]; nxt += 1
        pos = torch.arange(n)
        slots.append(bt[b, pos // PAGE].long() * PAGE + pos % PAGE)
        srcs.append(torch.randn(n, ld, dtype=torch.bfloat16))
    src, slot = torch.cat(srcs), torch.cat(slots)
    q = torch.randn(B, Hq * D, dtype=torch.bfloat16)
    outs = {}
    for d, c in caches.items():
        c.append(0, src.to(d), Hq * D, (Hq + Hkv) * D, slot.to(d))
        outs[d] = c.decode(0, q.to(d), bt.to(d), lens.to(d), Hq).float().cpu()
    torch.cuda.synchronize()
    # the stored (quantised) caches agree, so decode differences are kernel arithmetic only
    kd = (caches["cpu"].k[0].dequant() - caches["cuda"].k[0].dequant().cpu()).abs().max().item()
    assert kd < (0.02 if mode == "bf16" else 0.6), kd
    assert (outs["cpu"] - outs["cuda"]).abs().max().item() < (2e-2 if mode == "bf16" else 0.12)
    # and against an unquantised fp32 reference the error stays within the format's budget
    G = Hq // Hkv
    for b in range(B):
        n = int(lens[b])
        kk = srcs[b][:, Hq * D:(Hq + Hkv) * D].float().view(n, Hkv, D)
        vv = srcs[b][:, (Hq + Hkv) * D:].float().view(n, Hkv, D)
        s = torch.einsum("hgd,nhd->hgn", q[b].float().view(Hkv, G, D), kk) / math.sqrt(D)
        ref = torch.einsum("hgn,nhd->hgd", torch.softmax(s, -1), vv).reshape(-1)
        tol = {"bf16": 3e-2, "fp8": 0.15, "q4": 0.5}[mode]
        assert (outs["cuda"][b] - ref).abs().max().item() < tol


@pytest.mark.parametrize("mode", ["bf16", "fp8", "q4"])
@pytest.mark.parametrize("Hkv,D,n", [(2, 64, 100), (1, 128, 33), (4, 128, 256)])
def test_kv_gather_matches_host_dequant(mode, Hkv, D, n):
    """The gather kernel returns the first n cached tokens of a sequence as contiguous bf16 rows: identical to the host
    statement (dequantise the pool, pick the sequence's pages) after its one rounding to bf16."""
    pages = 40
    cache = PagedKVCache(1, pages, Hkv, D, mode, "cuda")
    npg = (n + PAGE - 1) // PAGE
    pg = torch.randperm(pages)[:npg].to(torch.int32)
    pos = torch.arange(n)
    slots = (pg[pos // PAGE].long() * PAGE + pos % PAGE).cuda()
    src = torch.randn(n, 2 * Hkv * D, device="cuda", dtype=torch.bfloat16)
    cache.append(0, src, 0, Hkv * D, slots)
    k, v = cache.gather(0, pg.cuda(), n)
    torch.cuda.synchronize()
    _lib.check_status()
    K = cache.k[0].dequant()[pg.long().cuda()].reshape(-1, Hkv * D)[:n].to(torch.bfloat16)
    V = cache.v[0].dequant()[pg.long().cuda()].reshape(-1, Hkv * D)[:n].to(torch.bfloat16)
    assert torch.equal(k, K) and torch.equal(v, V)
    tol = {"bf16": 0.0, "fp8": 0.3, "q4": 0.6}[mode]
    assert (k.float() - src[:, :Hkv * D].float()).abs().max().item() <= tol


def test_sampling_distribution_and_greedy():
    V, B = 1000, 4
    logits = torch.randn(B, V) * 2
    dev = "cuda"
    lg = logits.to(dev)
    # greedy rows
    t = torch.zeros(B, device=dev); k = torch.zeros(B, dtype=torch.int32, device=dev); p = torch.ones(B, device=dev)
    ids = S.sample(lg, t, k, p)
    assert torch.equal(ids.cpu(), logits.argmax(-1))
    # filtered sampling: every draw lies in the filtered support; empirical frequencies follow the target
    t = torch.full((B,), 0.8, device=dev); k = torch.full((B,), 20, dtype=torch.int32, device=dev)
    p = torch.full((B,), 0.9, device=dev)
    counts = torch.zeros(B, V)
    n = 4000
    for step in range(n):
        ids = S.sample(lg, t, k, p, seed=7, step=step).cpu()
        counts[torch.arange(B), ids] += 1
    for b in range(B):
        target = S._filtered_probs(logits[b], 0.8, 20, 0.9, 1.0, None)
        support = target > 0
        assert counts[b][~support].sum() <= 0.01 * n   # bisection edge may admit a boundary token
        freq = counts[b] / n
        assert (freq - target).abs().max().item() < 0.04
    torch.cuda.synchronize()
    _lib.check_status()


def test_repetition_penalty_and_bf16():
    V = 512
    logits = torch.zeros(1, V); logits[0, 5] = 5.0; logits[0, 9] = 4.9
    hist = torch.full((1, 8), -1, dtype=torch.int32); hist[0, 0] = 5; hist[0, 3] = 5
    t = torch.zeros(1, device="cuda"); k = torch.zeros(1, dtype=torch.int32, device="cuda"); p = torch.ones(1, device="cuda")
    r = torch.full((1,), 1.5, device="cuda")
    ids = S.sample(logits.bfloat16().cuda(), t, k, p, r, hist.cuda())
    assert int(ids[0]) == 9
