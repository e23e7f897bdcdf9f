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
