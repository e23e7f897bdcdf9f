"""Continuous-batching engine against full-sequence recomputation (token-exact for greedy decoding),
prefix reuse, page accounting, priorities, and KV quantisation error budgets.  Runs on CPU; the GPU
variant repeats the parity check with the kernels."""
import pytest
import torch

from transformers_fusion_b200.inference.engine import EngineConfig, InferenceEngine
from transformers_fusion_b200.inference.sampler import SamplerConfig
from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel

GREEDY = SamplerConfig(temperature=0.0, top_k=0, top_p=1.0)


def _model(device="cpu", dtype=torch.float32, **kw):
    base = dict(vocab_size=200, hidden_size=128, num_layers=2, num_heads=2, num_kv_heads=1, ffn_hidden_size=192,
                max_seq_len=256, init_std=0.08)
    base.update(kw)
    return DenseModel(TransformerConfig(**base), device=device, dtype=dtype, seed=4)


def _naive_greedy(model, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        logits = model(torch.tensor([ids], device=model.tok_embeddings.device))
        ids.append(int(logits[0, -1].float().argmax()))
    return ids[len(prompt):]


def test_engine_matches_recompute_cpu():
    m = _model()
    eng = InferenceEngine(m, None, EngineConfig(max_batch=4, num_pages=64))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (5, 17, 33, 40, 9)]
    outs = eng.generate_batch(prompts, max_tokens=12, sampling=GREEDY)
    for p, o in zip(prompts, outs):
        assert o == _naive_greedy(m, p, 12)
    assert eng.cache.allocator.num_free + (len(eng.prefix.table) if eng.prefix else 0) == 64 or eng.prefix.table
    assert not eng.has_pending()


def test_prefix_cache_reuses_pages_and_keeps_results():
    m = _model()
    base = torch.randint(3, 200, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    a, b = base + [7, 8, 9], base + [10, 11]
    cold = InferenceEngine(m, None, EngineConfig(num_pages=64, enable_prefix_cache=False))
    ref = cold.generate_batch([a, b], 8, GREEDY)
    warm = InferenceEngine(m, None, EngineConfig(num_pages=64, enable_prefix_cache=True, max_batch=1))
    got = warm.generate_batch([a, b], 8, GREEDY)
    assert got == ref
    assert warm.stats.prefix_hit_tokens == 32      # two whole pages of the shared prefix


def test_priority_order_and_page_exhaustion():
    m = _model()
    eng = InferenceEngine(m, None, EngineConfig(max_batch=1, num_pages=8, enable_prefix_cache=False))
    lo = eng.add_request([5] * 10, 4, GREEDY, priority=0)
    hi = eng.add_request([6] * 10, 4, GREEDY, priority=5)
    order = []
    while eng.has_pending():
        for r in eng.step():
            order.append(r.id)
    assert order == [hi.id, lo.id]
    assert eng.cache.allocator.num_free == 8


@pytest.mark.parametrize("mode,tol", [("fp8", 0.25), ("q4", 0.9)])
def test_quantised_kv_stays_close(mode, tol):
    m = _model()
    prompt = torch.randint(3, 200, (48,), generator=torch.Generator().manual_seed(2)).tolist()
    ref = InferenceEngine(m, None, EngineConfig(num_pages=32))
    q = InferenceEngine(m, None, EngineConfig(num_pages=32, kv_mode=mode))
    for e in (ref, q):
        r = e.add_request(prompt, 1, GREEDY)
        e.step()
    k0 = ref.cache.k[0].dequant()
    k1 = q.cache.k[0].dequant()
    used = k0.abs().sum((1, 2, 3)) > 0
    err = (k0[used] - k1[used]).abs().max().item() / k0[used].abs().max().item()
    assert err < tol * 0.2, err


@pytest.mark.gpu
def test_engine_matches_recompute_gpu():
    m = _model("cuda", torch.bfloat16, hidden_size=256, num_heads=4, num_kv_heads=2)
    eng = InferenceEngine(m, None, EngineConfig(max_batch=8, num_pages=128))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (5, 17, 130, 40)]
    outs = eng.generate_batch(prompts, max_tokens=8, sampling=GREEDY)
    agree = 0
    for p, o in zip(prompts, outs):
        ref = _naive_greedy(m, p, 8)
        agree += sum(int(x == y) for x, y in zip(o, ref))
    assert agree >= 28, agree      # bf16 paths differ in rounding; near-ties may flip a token


@pytest.mark.gpu
@pytest.mark.parametrize("kv_mode", ["bf16", "fp8"])
def test_prefix_cache_suffix_prefill_gpu(kv_mode):
    """A prompt whose first pages are cached: the suffix runs through the KV gather + tensor-core attention path and must
    give the tokens of an engine that prefills the whole prompt (bf16 rounding may flip a near-tie).  With an fp8 cache the
    two engines legitimately differ - the cold one attends over the exact prompt keys, the warm one over the fp8-rounded
    prefix - so only the first tokens are compared there."""
    m = _model("cuda", torch.bfloat16, hidden_size=256, num_heads=4, num_kv_heads=2)
    base = torch.randint(3, 200, (200,), generator=torch.Generator().manual_seed(1)).tolist()
    a, b = base + [7, 8, 9], base + list(range(10, 50))
    cold = InferenceEngine(m, None, EngineConfig(num_pages=128, enable_prefix_cache=False, kv_mode=kv_mode))
    ref = cold.generate_batch([a, b], 8, GREEDY)
    warm = InferenceEngine(m, None, EngineConfig(num_pages=128, enable_prefix_cache=True, max_batch=1, kv_mode=kv_mode))
    got = warm.generate_batch([a, b], 8, GREEDY)
    assert warm.stats.prefix_hit_tokens == 192
    agree = sum(int(x == y) for o, r in zip(got, ref) for x, y in zip(o, r))
    if kv_mode == "bf16":
        assert agree >= 12, (got, ref)
    else:
        assert all(len(o) == 8 for o in got) and agree >= 2, (got, ref)


def test_pipelined_schedule_on_cpu():
    """The pipelined schedule (launch first, read the previous step's tokens afterwards) run on the CPU, where arithmetic is
    deterministic: token-for-token the outputs of the synchronous schedule, with more requests than batch slots, sequences
    that end on a stop token (seen one step late), and every page returned at the end."""
    m = _model()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (5, 17, 60, 40, 9, 33, 21, 12)]

    def run(pipeline, stops):
        eng = InferenceEngine(m, None, EngineConfig(max_batch=3, num_pages=128, pipeline_decode=pipeline, enable_prefix_cache=False))
        reqs = [eng.add_request(p, max_tokens=10 + (i % 3), sampling=GREEDY, stop_ids=stops.get(i, ())) for i, p in enumerate(prompts)]
        steps = 0
        while eng.has_pending():
            eng.step()
            steps += 1
        assert eng.cache.allocator.num_free == 128
        return [r.out for r in reqs], steps
    base, n0 = run(False, {})
    pipe, n1 = run("force", {})
    assert pipe == base and [len(o) for o in base] == [10 + (i % 3) for i in range(len(prompts))]
    stops = {i: (o[4],) for i, o in enumerate(base) if i % 2 == 0}
    sync, _ = run(False, stops)
    pipe, _ = run("force", stops)
    assert pipe == sync and any(len(o) < 10 for o in sync)
    for i, o in enumerate(sync):
        if i in stops:
            assert o.index(stops[i][0]) == len(o) - 1


@pytest.mark.gpu
def test_pipelined_decode_matches_synchronous_gpu():
    """Launching a decode step before the previous step's tokens are read must not change anything the caller sees: same
    tokens for every request, also when sequences end early on a stop token (seen one step late by the scheduler), when
    requests are admitted while others decode, and with more requests than batch slots."""
    m = _model("cuda", torch.bfloat16, hidden_size=256, num_heads=4, num_kv_heads=2)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (5, 17, 60, 40, 9, 33, 21, 12, 50, 7)]

    def run(pipeline, stops):
        eng = InferenceEngine(m, None, EngineConfig(max_batch=4, num_pages=256, pipeline_decode=pipeline, enable_prefix_cache=False))
        reqs = [eng.add_request(p, max_tokens=12 + (i % 3), sampling=GREEDY, stop_ids=stops.get(i, ())) for i, p in enumerate(prompts)]
        steps = 0
        while eng.has_pending():
            eng.step()
            steps += 1
        assert eng.cache.allocator.num_free == 256, "every page must be back after the last request"
        return [r.out for r in reqs], steps
    def agreement(a, b):
        same = sum(int(x == y) for o, r in zip(a, b) for x, y in zip(o, r))
        return same / max(1, sum(min(len(o), len(r)) for o, r in zip(a, b)))
    base, _ = run(False, {})
    pipe, _ = run(True, {})
    assert [len(o) for o in pipe] == [len(o) for o in base] == [12 + (i % 3) for i in range(len(prompts))]
    assert agreement(pipe, base) >= 0.9, (pipe, base)        # split-K sums are atomic: near-ties may flip a token
    # stop tokens taken from the outputs themselves: those sequences end early, exactly at the stop token
    stops = {i: (o[3],) for i, o in enumerate(base) if i % 2 == 0}
    sync, n_sync = run(False, stops)
    pipe, n_pipe = run(True, stops)
    for outs in (sync, pipe):
        for i, o in enumerate(outs):
            if i in stops and stops[i][0] in o:
                assert o.index(stops[i][0]) == len(o) - 1, (i, o)      # nothing is emitted after the stop token
    assert any(len(o) < 12 for o in pipe) and agreement(pipe, sync) >= 0.9
    assert n_pipe <= n_sync + 4


def test_engine_with_packed_weights_matches_dequantised_model():
    """Serving from int8-packed weights must give the tokens of a model whose weights are the dequantised values."""
    import torch
    from transformers_fusion_b200.inference.engine import EngineConfig, InferenceEngine
    from transformers_fusion_b200.inference.sampler import SamplerConfig
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.quant import wq
    cfg = TransformerConfig(vocab_size=128, hidden_size=64, num_layers=2, num_heads=4, ffn_hidden_size=128, max_seq_len=64)
    m = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0)
    eng = InferenceEngine(m, None, EngineConfig(num_pages=32, weight_format="int8", weight_group=32))
    assert len(eng.packed) == 8
    out_q = eng.generate_batch([[5, 6, 7, 8]], 8, SamplerConfig(0.0))[0]
    m2 = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0)
    for i, l in enumerate(m2.layers):
        for name in ("qkv", "o", "gate_up", "down"):
            getattr(l, name).data.copy_(wq.dequant(eng.packed[f"layers.{i}.{name}"]))
    out_ref = InferenceEngine(m2, None, EngineConfig(num_pages=32)).generate_batch([[5, 6, 7, 8]], 8, SamplerConfig(0.0))[0]
    assert out_q == out_ref


@pytest.mark.gpu
@pytest.mark.parametrize("weights", ["", "int8"])
def test_decode_graph_replay_matches_eager(weights):
    """Captured decode steps (batch buckets 1, 2, 4 as requests finish at different lengths) give the eager tokens."""
    m = _model("cuda", torch.bfloat16, hidden_size=256, num_heads=4, num_kv_heads=2)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (9, 33, 70)]
    outs = []
    for graph in (False, True):
        eng = InferenceEngine(m, None, EngineConfig(max_batch=8, num_pages=128, cuda_graph=graph, weight_format=weights,
                                                    enable_prefix_cache=False))
        reqs = [eng.add_request(p, max_tokens=mt, sampling=GREEDY) for p, mt in zip(prompts, (4, 9, 14))]
        while eng.has_pending():
            eng.step()
        outs.append([r.out for r in reqs])
        if graph:
            assert sorted(eng._graphs) == [1, 2, 4]
    assert outs[0] == outs[1]


def test_batched_prefill_matches_one_by_one():
    """Prompts of different lengths prefilled together (padded) give the tokens of one-by-one prefill, and the padded rows
    leave no trace in the cache (page accounting is identical)."""
    m = _model()
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (5, 33, 18, 64, 7)]
    res = []
    for bp in (False, True):
        eng = InferenceEngine(m, None, EngineConfig(max_batch=8, num_pages=64, batch_prefill=bp, max_prefill_tokens=150,
                                                    enable_prefix_cache=False))
        outs = eng.generate_batch(prompts, max_tokens=6, sampling=GREEDY)
        res.append((outs, eng.cache.allocator.num_free, eng.stats.prompt_tokens))
    assert res[0] == res[1]


def _moe_model(device="cpu", dtype=torch.float32):
    from transformers_fusion_b200.models.config import MoEConfig
    from transformers_fusion_b200.models.moe import MoEModel
    cfg = MoEConfig(vocab_size=200, hidden_size=128, num_layers=2, num_heads=2, num_kv_heads=1, ffn_hidden_size=192, max_seq_len=256,
                    init_std=0.08, num_experts=4, top_k=2, expert_hidden_size=128)
    return MoEModel(cfg, device=device, dtype=dtype, seed=5)


def test_engine_serves_moe_model_cpu():
    m = _moe_model()
    eng = InferenceEngine(m, None, EngineConfig(max_batch=4, num_pages=64))
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (6, 21)]
    outs = eng.generate_batch(prompts, max_tokens=6, sampling=GREEDY)
    for p, o in zip(prompts, outs):
        assert o == _naive_greedy(m, p, 6)


@pytest.mark.gpu
def test_engine_serves_moe_model_gpu():
    m = _moe_model("cuda", torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 200, (n,), generator=g).tolist() for n in (6, 21, 40)]
    outs = []
    for graph in (False, True):
        eng = InferenceEngine(m, None, EngineConfig(max_batch=4, num_pages=64, cuda_graph=graph))
        outs.append(eng.generate_batch(prompts, max_tokens=6, sampling=GREEDY))
    assert outs[0] == outs[1]
    agree = sum(int(a == b) for p, o in zip(prompts, outs[0]) for a, b in zip(o, _naive_greedy(m, p, 6)))
    assert agree >= 15, agree
