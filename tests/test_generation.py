"""Generators, speculative decoding (must reproduce the target's greedy output), grammar masks, batcher, embeddings."""
import pytest
import torch

from transformers_fusion_b200.inference import generation as G
from transformers_fusion_b200.inference.sampler import SamplerConfig
from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.tokenizer import ByteTokenizer


def model(seed, layers=2, hidden=64):
    cfg = TransformerConfig(vocab_size=259, hidden_size=hidden, num_layers=layers, num_heads=4, ffn_hidden_size=128, max_seq_len=96)
    return DenseModel(cfg, device="cpu", dtype=torch.float32, seed=seed)


def test_generator_and_streaming():
    m, tok = model(0), ByteTokenizer()
    g = G.Generator(m, tok)
    res = g.generate_full("hello", SamplerConfig(temperature=0.0, max_tokens=8))
    assert len(res.tokens) <= 8 and res.tokens_per_sec > 0 and not res.truncated
    assert g.generate_tokens(tok.encode("hello"), SamplerConfig(temperature=0.0, max_tokens=8)) == res.tokens
    ev = []
    sg = G.StreamingGenerator(m, tok)
    sg.set_event_handler(lambda k, p: ev.append((k, p)))
    text = sg.generate("hello", G.StreamingConfig(SamplerConfig(temperature=0.0), max_tokens=8))
    kinds = [k for k, _ in ev]
    assert kinds[0] == "START" and kinds[-1] == "COMPLETE" and kinds.count("TOKEN") == len([t for t in sg.output_ids() if t != tok.eos_id])
    assert sg.output_ids() == res.tokens and isinstance(text, str)
    # stop string: cut at the first occurrence
    first_piece = next(p["text"] for k, p in ev if k == "TOKEN" and p["text"])
    ev.clear()
    out = sg.generate("hello", G.StreamingConfig(SamplerConfig(temperature=0.0), max_tokens=8, stop_strings=[first_piece]))
    assert ev[-1][0] == "STOP" and first_piece not in out


def test_speculative_greedy_equals_target():
    target, draft = model(0, layers=3), model(1, layers=1)
    prompt = ByteTokenizer().encode("speculate")
    ref = G.Generator(target, ByteTokenizer()).generate_tokens(prompt, SamplerConfig(temperature=0.0, max_tokens=24))
    sd = G.SpeculativeDecoder(target, draft, gamma=3)
    out = sd.generate(prompt, 24, SamplerConfig(temperature=0.0))
    assert out == ref[:len(out)] and len(out) == 24
    assert sd.stats.proposed > 0 and sd.stats.target_passes < 24 + 2
    # a perfect draft (the target itself) is always accepted: ~gamma+1 tokens per target pass
    sd2 = G.SpeculativeDecoder(target, target, gamma=4, adaptive=False)
    out2 = sd2.generate(prompt, 24, SamplerConfig(temperature=0.0))
    assert out2 == ref[:24] and sd2.stats.acceptance_rate == 1.0 and sd2.stats.tokens_per_target_pass > 3.5
    # sampling mode runs and respects the length
    assert len(G.SpeculativeDecoder(target, draft, gamma=2, seed=3).generate(prompt, 10, SamplerConfig(0.8, 20, 0.95))) == 10
    t = G.TreeDecoder(target, target, branching=2, depth=2).step(prompt)
    assert t == ref[:3]


def test_grammar_masks():
    ok = G.GrammarDecoder.json_prefix_ok
    for s in ['', '{', '{"a', '{"a": ', '{"a": [1, 2.5e', '{"a": tr', '[{"x": null}, "s"]', '  {"k": -0.1}']:
        assert ok(s), s
    for s in ['}', '{"a" 1', '[1,,', '{"a": 01', '{"a": 1}}', 'tru3', '[1 2']:
        assert not ok(s), s
    tok = ByteTokenizer()
    gd = G.GrammarDecoder(tok, 259, "json")
    m = gd.mask('{"a": ')
    allowed = {tok.decode([i]) for i in m.nonzero().reshape(-1).tolist()}
    assert {'"', '1', '[', '{', 't', '-', ' '} <= allowed and 'x' not in allowed and '}' not in allowed
    rg = G.GrammarDecoder(tok, 259, "regex", pattern=r"(yes|no)!?")
    m = rg.mask("ye")
    assert {tok.decode([i]) for i in m.nonzero().reshape(-1).tolist()} == {"s"}
    logits = torch.zeros(259)
    logits[tok.encode("q")[0]] = 5.0
    out = rg.constrain(logits, "", top=4)
    assert set(torch.isfinite(out).nonzero().reshape(-1).tolist()) == {tok.encode("y")[0], tok.encode("n")[0]}


def test_batcher_embeddings_lowprec():
    b = G.DynamicBatcher(max_batch=3, window_s=0.01)
    assert b.next_batch(0.01) is None
    for i, t in enumerate(([1, 2, 3], [4], [5, 6], [7])):
        b.submit(t, tag=i)
    ids, lens, tags = b.next_batch()
    assert ids.tolist() == [[1, 2, 3], [0, 0, 4], [0, 5, 6]] and lens == [3, 1, 2] and tags == [0, 1, 2]
    assert b.next_batch()[2] == [3]
    m, tok = model(0), ByteTokenizer()
    ep = G.EmbeddingEndpoint(m, tok)
    e = ep.embed(["abc", "abd", "zzzzzz"])
    assert e.shape == (3, 64) and torch.allclose(e.norm(dim=1), torch.ones(3), atol=1e-5)
    rr = G.Reranker(ep).rerank("abc", ["zzzzzz", "abc", "abd"])
    assert rr[0][0] == 1 and rr[0][1] == pytest.approx(1.0, abs=1e-5)
    w = torch.randn(32, 48)
    q = G.INT8Inference(w)
    x = torch.randn(5, 48)
    assert q.error(w) <= float(w.abs().amax(1).max()) / 127 and (q.forward(x) - x @ w.t()).abs().max() < 0.5
    sh0, sh1 = G.ModelShard(m, 0, 1), G.ModelShard(m, 1, 2)
    ids = torch.randint(0, 259, (2, 8))
    logits = sh1.forward(sh0.forward(ids, 2, 8), 2, 8)
    assert torch.allclose(logits.view(2, 8, -1), m.forward(ids).detach(), atol=1e-4)


def test_reference_named_inference_helpers():
    """Sampler verbs, tree decoding loop, batched generation, embeddings / reranking scores, speculative counters,
    prefix-cache verbs, the block pool and the compressed-KV accessors."""
    import torch
    from transformers_fusion_b200.inference import generation as G
    from transformers_fusion_b200.inference.engine import PrefixCache
    from transformers_fusion_b200.inference.kv_cache import PAGE, PageAllocator
    from transformers_fusion_b200.inference.kv_extras import CompressedKVCache
    from transformers_fusion_b200.inference.sampler import Sampler, SamplerConfig
    from transformers_fusion_b200.inference.speculative_extras import InferenceMemoryPool
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    s = Sampler(SamplerConfig(temperature=1.0, top_k=3, top_p=1.0, repetition_penalty=2.0))
    z = torch.tensor([4.0, 3.0, -2.0, 1.0, 0.5])
    assert s.greedy(z) == 0 and torch.allclose(s.apply_temperature(z, 2.0), z / 2)
    pen = s.apply_repetition_penalty(z, [0, 2], 2.0)
    assert pen.tolist() == [2.0, 3.0, -4.0, 1.0, 0.5]
    s.set_seed(7)
    draws = {s.sample_top_k(z, 2) for _ in range(40)}
    assert draws <= {0, 1} and len(draws) == 2
    assert {s.sample_top_p(z, 0.5) for _ in range(20)} == {0}
    assert s.sample(z, history=[0]) in (0, 1, 3)                    # the penalty demotes token 0 but keeps it in the top 3
    assert Sampler(SamplerConfig(temperature=0.0, repetition_penalty=4.0)).sample(z, history=[0]) == 1
    assert SamplerConfig(max_tokens=5000).effective_max_tokens("medium") == 2048 and SamplerConfig().effective_max_tokens() == 512
    assert G.StreamingConfig(max_tokens=999).effective_max_tokens("low") == 256
    tok = ByteTokenizer()
    cfg = TransformerConfig(vocab_size=260, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=64, max_seq_len=64)
    tgt, drf = DenseModel(cfg, dtype=torch.float32, seed=1), DenseModel(cfg, dtype=torch.float32, seed=1)
    out = G.TreeDecoder(tgt, drf, branching=2, depth=2).decode(tok.encode("ab"), 5)
    ids = tok.encode("ab")
    greedy = []
    for _ in range(5):
        with torch.no_grad():
            greedy.append(int(tgt(torch.tensor([ids + greedy]))[0, -1].argmax()))
    assert out == greedy                                             # identical draft: every tree step is accepted in full
    texts = G.DynamicBatcher(max_batch=4, model=tgt, tokenizer=tok).batch_generate(["ab", "hello"], 4)
    assert len(texts) == 2 and all(isinstance(t, str) for t in texts)
    ep = G.EmbeddingEndpoint(tgt, tok)
    assert ep.embed_batch(["a", "bc"]).shape == (2, 32)
    rr = G.Reranker(ep)
    sc = rr.score_batch("hello", ["hello", "zzzz"])
    assert abs(sc[0] - 1.0) < 1e-5 and rr.score("hello", "zzzz") == pytest.approx(sc[1], abs=1e-6) and sc[1] < sc[0]
    sd = G.SpeculativeDecoder(tgt, drf, gamma=2, adaptive=False)
    sd.generate(tok.encode("ab"), 6)
    assert sd.accepted_count() == sd.total_count() > 0 and sd.acceptance_rate() == 1.0 and sd.current_gamma() == 2.0
    assert not sd.used_uniform_draft_fallback()
    alloc = PageAllocator(8)
    pc = PrefixCache(alloc)
    toks = list(range(2 * PAGE + 3))
    pages = [alloc.alloc(), alloc.alloc()]
    pc.store(toks, pages)
    assert pc.match_prefix(toks) == 2 * PAGE and pc.match_prefix(toks[:PAGE + 1]) == PAGE and pc.match_prefix([9] * 40) == 0
    assert pc.get_cache(toks) == pages and alloc.refs[pages[0]] == 3
    pool = InferenceMemoryPool.of_blocks(1024, 2)
    a, b = pool.alloc(), pool.alloc()
    assert {a, b} == {0, 1} and pool.alloc() is None and pool.used == 2048
    pool.free(a)
    assert pool.alloc() == a
    with pytest.raises(ValueError):
        pool.free(b), pool.free(b)
    kv = CompressedKVCache(2, 32, 8)
    k, v = torch.randn(3, 2, 32), torch.randn(3, 2, 32)
    kv.append(k, v)
    K, V = kv.get()
    assert torch.equal(kv.get_k(1), K[1]) and torch.equal(kv.get_v(2), V[2]) and kv.size() == 3
    kv.clear()
    assert kv.size() == 0
    with pytest.raises(IndexError):
        kv.get_k(0)


def test_attention_variants_against_plain_statement():
    import math
    import torch
    from transformers_fusion_b200.inference.attention_variants import (ALiBi, GroupedQueryAttention, MultiQueryAttention,
                                                                     SlidingWindowAttention, compute_logprobs)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 10, 32, generator=g)

    def plain(m, bias=None):
        B, S, _ = x.shape
        H, Hkv, D = m.n_heads(), m.n_kv_heads(), m.head_dim
        q = (x @ m.w_q.t()).view(B, S, H, D).transpose(1, 2)
        k = (x @ m.w_k.t()).view(B, S, Hkv, D).transpose(1, 2).repeat_interleave(H // Hkv, 1)
        v = (x @ m.w_v.t()).view(B, S, Hkv, D).transpose(1, 2).repeat_interleave(H // Hkv, 1)
        s = q @ k.transpose(-1, -2) / math.sqrt(D)
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
        if bias is not None:
            s = s + bias
        return (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, S, H * D) @ m.w_o.t()
    gqa = GroupedQueryAttention(32, 4, 2, seed=1)
    assert torch.allclose(gqa(x), plain(gqa), atol=1e-5) and gqa.w_k.shape == (16, 32)
    mqa = MultiQueryAttention(32, 4, seed=2)
    assert mqa.n_kv_heads() == 1 and torch.allclose(mqa(x), plain(mqa), atol=1e-5)
    swa = SlidingWindowAttention(32, 4, window_size=3, seed=3)
    i, j = torch.arange(10)[:, None], torch.arange(10)[None, :]
    assert torch.allclose(swa(x), plain(swa, torch.where(i - j >= 3, float("-inf"), 0.0)), atol=1e-5)
    wide = SlidingWindowAttention(32, 4, window_size=64, seed=3)
    assert torch.allclose(wide(x), plain(wide), atol=1e-5)          # a window longer than the sequence changes nothing
    al = ALiBi(4, 32, seed=4)
    assert al.slopes.tolist() == pytest.approx([0.25, 0.0625, 0.015625, 0.00390625])
    bias = al.build_alibi_bias(10, 10)
    assert bias.shape == (4, 10, 10) and float(bias[0, 5, 3]) == -0.5 and float(bias[0, 3, 5]) == 0.0
    assert torch.allclose(al(x), plain(al, bias), atol=1e-5) and len(ALiBi.compute_slopes(6)) == 6
    lp = compute_logprobs(torch.randn(3, 7, generator=g), [1, 2, 3])
    assert len(lp) == 3 and len(lp[0]) == 7 and abs(sum(math.exp(v) for v in lp[0]) - 1.0) < 1e-5


def test_fp8_two_stage_forward_reduces_activation_rounding_error():
    from transformers_fusion_b200.inference.generation import FP8Inference
    from transformers_fusion_b200.quant import fp8
    torch.manual_seed(0)
    w, x = torch.randn(128, 256), torch.randn(16, 256)
    lin = FP8Inference(w)
    ref = x @ fp8.dequant(lin.qw, lin.sw, 128).t()               # exact activations, the same quantised weights
    e1 = (lin.forward(x).float() - ref).abs().mean()
    e2 = (lin.forward_two_stage(x).float() - ref).abs().mean()
    assert e2 < e1


def test_model_evaluator_run_all_on_cpu():
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.utils.metrics import ModelEvaluator
    m = DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=64, max_seq_len=32), device="cpu",
                   dtype=torch.float32, seed=0)
    ev = ModelEvaluator(m, batch_size=2)
    res = ev.run_all([int(i) % 64 for i in range(100)])
    assert [r.name for r in res] == ["perplexity", "accuracy"] and res[0].perplexity > 1.0 and 0.0 <= res[1].accuracy <= 1.0 and ev.results == res
