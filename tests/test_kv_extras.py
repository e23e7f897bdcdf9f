import pytest
import torch

from transformers_fusion_b200.inference import kv_extras as K


def test_page_table_levels():
    t2, t3 = K.PageTable(2), K.PageTable(3)
    assert t2.capacity_tokens() == 4096 * 4096 * 16 and t3.capacity_tokens() == 4096 ** 3 * 16
    t2.set(5, 50), t2.set(4096 * 4095 + 7, 77)
    assert t2.get(5) == 50 and t2.get(4096 * 4095 + 7) == 77 and t2.get(6) is None and t2.count == 2
    assert t2.pop(5) == 50 and t2.get(5) is None and t2.count == 1
    with pytest.raises(IndexError):
        t2.set(4096 * 4096, 1)
    t3.set(4096 * 4096 + 3, 9)
    assert t3.get(4096 * 4096 + 3) == 9


def test_spill_and_restore(tmp_path):
    st = K.TieredKVStore(2, 8, resident_pages=3, path=str(tmp_path / "kv.spill"))
    pages = {i: torch.randn(2, 16, 2, 8) for i in range(6)}
    for i, p in pages.items():
        st.write_page(i, p)
    assert st.stats["evictions"] == 3 and st.on_disk == {0, 1, 2} and st.table.get(0) is None and st.table.get(5) is not None
    st.prefetch([0])
    assert st.ensure_resident([0, 1]) and torch.equal(st.read_page(0), pages[0]) and torch.equal(st.read_page(1), pages[1])
    for i in range(6):                                      # everything survives being cycled through disk
        assert torch.equal(st.read_page(i), pages[i])
    assert st.stats["loads"] >= 3
    # a page that is neither resident nor on disk cannot become resident: bounded wait, no hang
    st.on_disk.add(99)
    st.file.truncate(0)
    st.q.put = lambda *_: None                                # the load request is lost on the way to the worker
    assert st.ensure_resident([99], timeout_ms=100) is False


def test_compressed_kv_and_flash_decoding():
    torch.manual_seed(0)
    c = K.CompressedKVCache(2, 64, 32)
    k, v = torch.randn(10, 2, 64), torch.randn(10, 2, 64)
    c.append(k[:6], v[:6]), c.append(k[6:], v[6:])
    kk, vv = c.get()
    assert kk.shape == (10, 2, 64) and c.bytes_per_token() == 2 * 2 * (16 + 4)
    cos = torch.nn.functional.cosine_similarity(kk.reshape(-1), k.reshape(-1), dim=0)
    assert cos > 0.75 and set(torch.unique(torch.sign(kk)).tolist()) <= {-1.0, 0.0, 1.0}
    q = torch.randn(4, 64)
    K_, V_ = torch.randn(50, 2, 64), torch.randn(50, 2, 64)
    ref = torch.empty(4, 64)
    for h in range(4):
        s = (K_[:, h // 2] @ q[h]) * 64 ** -0.5
        ref[h] = torch.softmax(s, 0) @ V_[:, h // 2]
    for splits in (1, 3, 7):
        assert torch.allclose(K.flash_decoding(q, K_, V_, splits), ref, atol=1e-5)


def test_budget_and_facades():
    b = K.ReasoningBudget.for_level("low")
    assert b.budget == 256 and b.consume(255) and not b.consume(1) and b.remaining() == 0
    from transformers_fusion_b200.inference.kv_cache import PagedKVCache
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    cache = PagedKVCache(1, 8, 2, 64, "bf16", "cpu")
    pa = K.PagedAttention(cache)
    blk = pa.alloc_block()
    assert cache.allocator.num_free == 7
    pa.free_block(blk)
    assert cache.allocator.num_free == 8
    m = DenseModel(TransformerConfig(vocab_size=259, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=64),
                   device="cpu", dtype=torch.float32, seed=0)
    cb = K.ContinuousBatching(m, ByteTokenizer(), max_batch=2, num_pages=32)
    for i in range(3):
        cb.add_request(K.BatchRequest([5 + i, 6, 7], 4, id=100 + i))
    done = []
    while cb.has_pending():
        done += cb.step()
    assert sorted(r.id for r in done) == [100, 101, 102] and all(len(r.tokens) <= 4 for r in done)


def test_q4_kv_cache_lloyd_max_codebooks():
    """4-bit KV with a trained 16-entry codebook per block: round trip error, nibble order, ratio, range reads."""
    import torch
    from transformers_fusion_b200.inference.kv_extras import Q4KVCache
    torch.manual_seed(0)
    H, D, L = 4, 32, 2
    c = Q4KVCache(L, 64, H, D, block_size=64)
    k = torch.randn(1, H, 10, D)
    v = torch.randn(1, H, 10, D) * 3 + 1
    c.append(0, k, v)
    c.append(0, k[:, :, :3], v[:, :, :3])
    assert c.context_len() == 13
    kk, vv = c.get_range(0, 0, 10)
    assert kk.shape == (1, H, 10, D)
    for a, b in ((kk, k), (vv, v)):
        nmse = float(((a - b) ** 2).sum() / (b ** 2).sum())
        assert nmse < 0.02, nmse                      # 16 trained levels per 64 values
    # a uniform 16-level grid over the block range (the Lloyd-Max starting point) must be no better than the trained codebook
    flat = k.permute(2, 1, 0, 3).reshape(-1, 64)
    pk, cb = Q4KVCache.quantize_blocks(flat, iters=0)
    pk2, cb2 = Q4KVCache.quantize_blocks(flat, iters=20)
    e0 = float(((Q4KVCache.dequantize_blocks(pk, cb) - flat) ** 2).sum())
    e1 = float(((Q4KVCache.dequantize_blocks(pk2, cb2) - flat) ** 2).sum())
    assert e1 < e0
    # nibble order: element 0 in the low nibble
    one = torch.zeros(1, 64); one[0, 0] = 5.0
    pk, cb = Q4KVCache.quantize_blocks(one)
    assert float(cb.float()[0, int(pk[0, 0]) & 0xF]) > 4.0
    assert abs(c.compression_ratio() - 4.0) < 1e-6      # 32 index + 32 codebook bytes per 64 fp32 values
    k2, _ = c.get_range(0, 10, 13)
    assert k2.shape == (1, H, 3, D) and float((k2 - k[:, :, :3]).abs().max()) < 1.0
    c.resize(128)
    assert c.max_seq_len() == 128 and c.get_all(0)[0].shape[2] == 13
    c.clear()
    assert c.context_len() == 0


def test_memory_efficient_attention_backward_and_stats():
    import math
    import torch
    from transformers_fusion_b200.inference.speculative_extras import MemoryEfficientAttention
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 3, 20, 8, generator=g) for _ in range(3))
    mea = MemoryEfficientAttention(block_q=8, block_k=4)
    with torch.no_grad():
        out = mea.forward(q, k, v)
    st = mea.last_softmax_stats()
    assert st["num_blocks"] > 0 and st["sum_val"] >= 1.0 and math.isfinite(st["max_val"])
    qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
    s = (qd @ kd.transpose(-1, -2)) / math.sqrt(8)
    s = s.masked_fill(torch.ones(20, 20, dtype=torch.bool).triu(1), float("-inf"))
    ref = torch.softmax(s, -1) @ vd
    assert torch.allclose(out, ref, atol=1e-5)
    go = torch.randn(ref.shape, generator=g)
    ref.backward(go)
    dq, dk, dv = mea.backward(go, q, k, v)
    assert torch.allclose(dq, qd.grad, atol=1e-4) and torch.allclose(dk, kd.grad, atol=1e-4) and torch.allclose(dv, vd.grad, atol=1e-4)
    # one tile of the running soft-max, twice, equals the soft-max over both key blocks
    sc = torch.randn(5, 6, generator=g)
    vv = torch.randn(6, 4, generator=g)
    m, l, o = torch.full((5,), -float("inf")), torch.zeros(5), torch.zeros(5, 4)
    for a in (0, 3):
        m, l, o = MemoryEfficientAttention.online_softmax_tile(sc[:, a:a + 3], m, l, o, vv[a:a + 3])
    assert torch.allclose(o / l[:, None], torch.softmax(sc, -1) @ vv, atol=1e-6)
    mea.set_config(block_size_q=16, max_context_tokens=1 << 10)
    assert mea.config() == {"block_size_q": 16, "block_size_kv": 4, "max_context_tokens": 1024}
    assert mea.forward_memory_bytes(1, 8, 4096, 64) < 4096 * 4096 * 4 * 8 and mea.backward_memory_bytes(1, 8, 4096, 64) > mea.forward_memory_bytes(1, 8, 4096, 64) / 4


def test_cache_init_forms_and_capacity():
    from transformers_fusion_b200.inference.kv_cache import PAGE, PagedKVCache
    from transformers_fusion_b200.inference.kv_extras import Q4KVCache
    c = PagedKVCache.init(2, 100, 2, 32, mode="bf16", device="cpu", sequences=3)
    pages = (100 + PAGE - 1) // PAGE
    assert c.num_pages == 3 * pages and c.logical_capacity() == 3 * pages * PAGE == c.max_seq_len()
    q = Q4KVCache(1, 8, 2, 32, block_size=32)
    assert q.init(2, 16, 2, 32, 64) is q and q.num_layers == 2 and q.k_idx[0].shape == (16 * 1, 32) and q.pos == [0, 0]
