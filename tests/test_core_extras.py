"""Core value types, thread-safety helpers, ranking metrics, speculative-decoding extras, tiled long-context attention."""
import math
import threading

import pytest
import torch

from transformers_fusion_b200.inference import speculative_extras as SX
from transformers_fusion_b200.inference.kv_cache import PageAllocator
from transformers_fusion_b200.utils import core as C, metrics as MX


def test_types():
    s = C.Shape(2, 3, 4)
    assert s.rank == 3 and s.numel() == 24 and s.strides() == (12, 4, 1) and C.Shape([5]).numel() == 5
    with pytest.raises(ValueError):
        C.Shape(*range(9))
    assert C.DType.U4.bits == 4 and C.DType.BF16.torch() == torch.bfloat16
    assert C.Status.OK() and not C.Status.error("x") and C.Status.error("bad").message == "bad"
    assert C.Config().seed == 42
    with pytest.raises(RuntimeError):
        C.quant_check(False, "boom")


def test_spsc_queue_between_threads():
    q = C.SPSCQueue(8)
    assert q.capacity == 8 and q.empty() and q.pop() is None
    got, N = [], 2000

    def consumer():
        while len(got) < N:
            v = q.pop()
            if v is not None:
                got.append(v)
    t = threading.Thread(target=consumer)
    t.start()
    i = 0
    while i < N:
        if q.push(i):
            i += 1
    t.join(10)
    assert got == list(range(N))
    for j in range(8):
        assert q.push(j)
    assert not q.push(99) and len(q) == 8


def test_shared_mutex_atomic_float_spinlock_counter():
    mu, state, seen = C.SharedMutex(), {"v": 0}, []

    def writer():
        for _ in range(200):
            with mu.unique():
                a = state["v"]
                state["v"] = a + 1

    def reader():
        for _ in range(200):
            with mu.shared():
                seen.append(state["v"])
    ts = [threading.Thread(target=f) for f in (writer, writer, reader, reader)]
    [t.start() for t in ts]
    [t.join(10) for t in ts]
    assert state["v"] == 400 and len(seen) == 400
    af, lock, total = C.AtomicFloat(), C.SpinLock(), {"n": 0}
    cnt = C.ThreadSafeCounter()

    def work():
        for _ in range(500):
            af.fetch_add(0.5)
            with lock:
                total["n"] += 1
            cnt.increment("steps")
    ts = [threading.Thread(target=work) for _ in range(4)]
    [t.start() for t in ts]
    [t.join(10) for t in ts]
    assert af.load() == 1000.0 and total["n"] == 2000 and cnt.get("steps") == 2000
    assert af.compare_exchange(1000.0, 1.0) and not af.compare_exchange(5.0, 2.0) and af.fetch_max(3.0) == 1.0 and af.load() == 3.0
    assert lock.try_lock() and not lock.try_lock()
    lock.unlock()
    cnt.reset("steps")
    assert cnt.snapshot() == {}


def test_ranking_metrics():
    assert MX.average_precision([0.9, 0.8, 0.7, 0.6], [1, 0, 1, 0]) == pytest.approx((1 + 2 / 3) / 2)
    assert MX.mean_average_precision([[0.9, 0.1], [0.2, 0.8], [0.5, 0.4]], [[1, 0], [1, 0], [0, 0]]) == pytest.approx((1 + 0.5) / 2)
    lg = torch.tensor([[0.1, 0.9, 0.5], [0.8, 0.1, 0.3]])
    assert MX.topk_accuracy(lg, [2, 2], 1) == 0.0 and MX.topk_accuracy(lg, [2, 2], 2) == 1.0


def test_speculation_plan_and_verifier():
    p = SX.SpeculationPlan.compute(0.8, 0.1)
    assert p.optimal_k == round(math.sqrt(2 / 0.2)) and p.speedup == pytest.approx((1 + 3 * 0.8) / (1 + 3 * 0.1))
    assert SX.Theorem13Result.compute(0.05, 0.1).speedup == 1.0
    d = torch.tensor([[0., 1], [1, 0], [0, 1], [1, 0]])
    t = torch.tensor([[0., 2], [3, 0], [5, 1], [1, 0]])
    r = SX.SmallBatchVerifier(8).verify(d, t)
    assert r.accepted == [True, True, False, False] and r.first_rejection_pos == 2 and r.total_accepted == 2
    assert SX.SmallBatchVerifier(1).verify(d, t).accepted == [True]


def test_kv_checkpoint_rewind_and_pool():
    alloc = PageAllocator(8)
    pages = [alloc.alloc() for _ in range(2)]              # 20 tokens -> 2 pages
    ck = SX.checkpoint_kv(pages, 20)
    pages += [alloc.alloc(), alloc.alloc()]                # drafting grew the sequence to 50 tokens
    assert alloc.num_free == 4
    assert SX.rewind_kv(alloc, pages, ck, 23) == 23        # 3 draft tokens accepted
    assert len(pages) == 2 and alloc.num_free == 6
    with pytest.raises(ValueError):
        SX.rewind_kv(alloc, pages, SX.KVCheckpoint(), 5)
    pool = SX.InferenceMemoryPool(1000)
    assert pool.reserve("a", 600) and not pool.reserve("b", 500) and pool.reserve("b", 400)
    assert pool.utilization() == 1.0 and pool.release("a") == 600 and pool.available() == 600 and pool.owners() == 1 and pool.peak == 1000


def test_tiled_attention_matches_dense_and_window():
    torch.manual_seed(0)
    H, S, d = 2, 150, 16
    q, k, v = (torch.randn(H, S, d) for _ in range(3))
    att = SX.MemoryEfficientAttention(32, 32)
    s = q @ k.transpose(-1, -2) / math.sqrt(d)
    causal = torch.tril(torch.ones(S, S, dtype=torch.bool))
    ref = torch.softmax(s.masked_fill(~causal, -float("inf")), -1) @ v
    assert torch.allclose(att.forward(q, k, v), ref, atol=1e-5)
    ref_full = torch.softmax(s, -1) @ v
    assert torch.allclose(att.forward(q, k, v, causal=False), ref_full, atol=1e-5)
    W, G = 40, 4
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    band = causal & ((j > i - W) | (j < G))
    ref_w = torch.softmax(s.masked_fill(~band, -float("inf")), -1) @ v
    assert torch.allclose(att.forward_block_sparse(q, k, v, W, G), ref_w, atol=1e-5)
    mem = att.memory_bytes(1 << 16, 8, 64)
    assert mem["tiled"] < mem["naive"] / 100
    with pytest.raises(ValueError):
        SX.MemoryEfficientAttention(max_context_tokens=100).forward(q, k, v)
    mg = SX.MultiGPUManager()
    assert mg.device_count() == len(mg.detect()) and mg.allocate_on(0, (2, 3)).shape == (2, 3)


def test_mapped_file_json_value_rate_limiter_and_aliases(tmp_path):
    p = tmp_path / "f.bin"
    p.write_bytes(bytes(range(50)))
    with C.MappedFile(str(p)) as mf:
        assert mf.size == 50 and mf.read(10, 5) == bytes(range(10, 15)) and len(mf.view()) == 50
        with pytest.raises(ValueError):
            mf.read(48, 5)
    j = C.JsonValue.parse('{"a": {"b": [1, 2.5, "x", true]}, "n": 3}')
    assert j.get_int("n") == 3 and j.get_float("a.b.1") == 2.5 and j.get_str("a.b.2") == "x" and j.get_bool("a.b.3") is True
    assert j.get("a.zz", "d") == "d" and j.get_int("a.b.2", 7) == 7 and j.is_object() and C.JsonValue.parse(j.dump()).get_int("a.b.0") == 1
    from transformers_fusion_b200.server.production import RateLimiter
    t = [0.0]
    rl = RateLimiter(rate=2.0, burst=3.0, clock=lambda: t[0])
    assert [rl.allow("ip") for _ in range(4)] == [True, True, True, False] and rl.allow("other")
    assert rl.retry_after("ip") == pytest.approx(0.5)
    t[0] = 1.0
    assert rl.allow("ip") and rl.allow("ip") and not rl.allow("ip")
    from transformers_fusion_b200.parallel.fsdp import GradientCheckpointManager, ZeROOptimizer, ZeroOptimizer
    assert ZeROOptimizer is not ZeroOptimizer and hasattr(ZeROOptimizer, "step_mixed") and hasattr(ZeroOptimizer, "reduce_scatter_grads")
    g = GradientCheckpointManager([100, 100, 400, 100], [1, 1, 2, 1])
    assert g.plan(1000) == [False] * 4 and g.plan(350) == [False, False, True, False] and g.saved_bytes() == 300
    assert g.recompute_overhead() == pytest.approx(0.4) and all(g.plan(0))
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.moe import MoEAllConfig, create_moe_variant
    base = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=48, max_seq_len=32, init_std=0.1)
    m = create_moe_variant("shared_expert", base, MoEAllConfig(num_experts=4, top_k=2, expert_hidden=32), dtype=torch.float32, seed=0)
    assert m.cfg.variant == "SHARED_EXPERT" and m.cfg.num_shared_experts == 1 and m(torch.randint(0, 64, (1, 8))).shape[-1] == 64
    with pytest.raises(ValueError):
        create_moe_variant("nope", base)
    from transformers_fusion_b200.agi.core import CodeGenSelfImprover, HPOptimizer, NeuralArchitectureSearch
    assert HPOptimizer().engine is not None and NeuralArchitectureSearch().engine is not None
    assert CodeGenSelfImprover().improve({"attention": 5.0}) is None     # hand-written kernels are not generated


def test_json_node_accessors_and_inferno_units():
    from transformers_fusion_b200.utils import core as C
    from transformers_fusion_b200.utils.inferno import InfernoCounter
    j = C.JsonValue.parse('{"n": 3, "f": 2.5, "s": "x", "b": true, "a": [1, "two", null], "o": {"k": 1}}')
    assert j["n"].as_int_checked() == 3 and j["f"].as_float() == 2.5 and j["n"].as_float() == 3.0 and j["s"].as_string_checked() == "x"
    assert j["b"].as_bool_checked() is True and j["missing"].is_null() and j.has("o") and not j.has("zz") and j["o"]["k"].int_val == 1
    assert [v.type for v in j["a"].arr] == [C.JsonValue.INT, C.JsonValue.STRING, C.JsonValue.NUL] and j["a"][1].str_val == "two"
    assert j["a"].at_or_null(9).is_null() and j["o"].obj["k"].as_int() == 1 and j["s"].is_string() and j["f"].is_number() and j["b"].is_bool()
    with pytest.raises(IndexError):
        j["a"][5]
    with pytest.raises(TypeError):
        j["s"].as_int_checked()
    with pytest.raises(TypeError):
        j["f"].as_int_checked()
    assert j["s"].as_int() == 0 and j["n"].as_string() == "" and C.JsonValue.parse(j.to_string())["a"][0].as_int() == 1
    bad, err = C.JsonValue.try_parse("{oops")
    assert bad.is_null() and err and C.json_escape_string('a"b\n') == 'a\\"b\\n'
    c = InfernoCounter()
    c.record("Q_4", 1000), c.record(9, 1000), c.record_mix("Q_MX_8_5", 1000), c.record(99, 5), c.record_iw(2.0, 1000)
    assert c.mean_info_weight() == pytest.approx((8.0 + 1.0 + 32.0 / 8.5 + 2.0) / 4) and c.ops == 8000
    c.ns = int(1e6)                                          # one millisecond
    assert c.elapsed_sec() == 1e-3 and c.gflops() == pytest.approx(8000 / 1e-3 / 1e9) == c.effective_gflops()
    raw = c.raw_ops_per_sec()
    assert c.minferno() == pytest.approx(raw / 1e6) and c.uinferno() == pytest.approx(raw / 1e9) and c.ninferno() == pytest.approx(raw / 1e12)
    assert c.pinferno() == pytest.approx(raw / 1e15) and c.best_unit() == "fInferno" and c.best_value() == pytest.approx(raw / 1e21 * 1e12)
    c.ops, c.ns = int(4e24), int(1e9)
    assert c.best_unit() == "Inferno" and c.best_value() >= 1.0
    c.reset()
    assert c.ops == 0 and c.mean_info_weight() == 1.0


def test_small_accessors_locks_counters_shapes_verifier_and_json_helpers():
    from transformers_fusion_b200.utils import core as C
    from transformers_fusion_b200.utils.hf_streamer import SimpleJSON
    from transformers_fusion_b200.inference import speculative_extras as SX
    from transformers_fusion_b200.server.production import RateLimiter
    m = C.SharedMutex()
    assert m.try_lock_shared() and m.try_lock_shared() and not m.try_lock()
    m.unlock_shared(), m.unlock_shared()
    assert m.try_lock() and not m.try_lock_shared() and not m.try_lock()
    m.unlock()
    assert m.try_lock_shared()
    c = C.ThreadSafeCounter()
    c.add(3), c.add(2, "x"), c.increment("x")
    assert c.total() == 6 and c.get("x") == 3 and C.Shape(2, 3, 4).to_string() == "[2, 3, 4]" and C.Shape().to_string() == "[]"
    doc = '{"a": {"id": 7, "name": "inner"}, "list": [{"name": "second"}], "tags": ["x", 1, "y"]}'
    assert SimpleJSON.find_string(doc, "name") == "inner" and SimpleJSON.find_string(doc, "id") == "" and SimpleJSON.find_string("{bad", "a") == ""
    assert SimpleJSON.find_all_strings_in_array('["x", 1, "y"]') == ["x", "y"] == SimpleJSON.find_all_strings_in_array(SimpleJSON.find_array(doc, "tags"))
    v = SX.SmallBatchVerifier(4)
    d = torch.eye(4)
    r8 = v.verify(d, d)
    v.set_format_index(3)                                         # Q_4: twice the information weight of Q_8
    r4 = v.verify(d, d)
    assert r8.total_accepted == 4 and r8.verify_inferno == pytest.approx(r8.verify_flops * 4 / 2) and r4.verify_inferno == pytest.approx(2 * r8.verify_inferno)
    g = SX.MultiGPUManager()
    assert g.detect_devices() == g.device_count() and not g.init_device(99) and g.device_name(99) == "cpu"
    t = torch.ones(8)
    g.free_on(0, t)
    assert t.numel() == 0
    now = [0.0]
    rl = RateLimiter(1.0, 3.0, clock=lambda: now[0])
    assert [rl.allow("a") for _ in range(4)] == [True, True, True, False]
    rl.set_limits(10.0, 1.0)
    now[0] += 1.0
    assert rl.max_requests_per_sec() == 10.0 and rl.burst_size() == 1.0 and [rl.allow("a") for _ in range(2)] == [True, False]


def test_status_rotary_object_replay_entry_and_loader_config(tmp_path):
    from transformers_fusion_b200.utils import core as C
    from transformers_fusion_b200.models.dense import RotaryEmbedding
    from transformers_fusion_b200.trainer.continual import CompressedReplayBuffer
    from transformers_fusion_b200.trainer.trainer import DataLoader, DataLoaderConfig
    assert C.Status.success() and C.Status.success().msg == "" and C.Status.error("bad").msg == "bad" and not C.Status.error("bad")
    r = RotaryEmbedding(8, 32)
    x = torch.randn(2, 3, 5, 8)
    ref = x.clone()
    half = 4
    pos = torch.arange(4, 9).float()
    inv = 10000.0 ** (-torch.arange(half).float() * 2 / 8)
    ang = pos[:, None] * inv[None]
    want = torch.cat([ref[..., :half] * ang.cos() - ref[..., half:] * ang.sin(), ref[..., half:] * ang.cos() + ref[..., :half] * ang.sin()], -1)
    assert r.apply(x, 4, 5) is x and torch.allclose(x, want, atol=1e-5) and r.attn_scale_mult() == 1.0
    y = RotaryEmbedding(8, 64, scaling_mode="yarn", scaling_factor=4.0, original_max_seq_len=16, yarn_attn_factor=1.0)
    assert y.attn_scale_mult() == pytest.approx(0.1 * math.log(4.0) + 1.0, rel=1e-6)
    b = CompressedReplayBuffer(8)
    b.insert(torch.arange(4.0), torch.ones(4), task_id=3)
    assert b.at(0).task_id == 3
    with pytest.raises(IndexError):
        b.at(1)
    p = tmp_path / "c.txt"
    p.write_text("abcdefghij" * 40)
    cfg = DataLoaderConfig(data_path=str(p), batch_size=2, seq_length=8, world_size=2, rank=1, seed=7)
    dl = DataLoader.from_config(cfg)
    assert dl.config() is cfg and dl.num_batches() == (400 - 1) // (2 * 8 * 2)
    ids, lab = dl.next_batch_with_labels()
    assert ids.shape == (2, 8) and torch.equal(ids[:, 1:], lab[:, :-1])
    plain = DataLoader(tokens=torch.arange(100), batch_size=2, seq_length=4)
    assert plain.config().batch_size == 2 and plain.config().seq_length == 4 and plain.config().shuffle_buffer == 0


def test_accumulating_metric_objects_and_scheduler_names():
    from transformers_fusion_b200.utils import metrics as M
    from transformers_fusion_b200.trainer import schedulers as S
    logits = torch.tensor([[2.0, 1.0, 0.0], [0.0, 1.0, 2.0], [0.0, 3.0, 1.0], [1.0, 0.0, 2.0]])
    tgt = torch.tensor([0, 1, 1, 0])
    a1, a2 = M.Accuracy(1), M.Accuracy(2)
    assert a1.update(logits, tgt) == 0.5 and a2.update(logits, tgt) == 1.0 and a1.update(torch.tensor([0, 1]), [0, 0]) == pytest.approx(3 / 6)
    assert (a1.correct(), a1.total(), a2.top_k()) == (3, 6, 2)
    a1.reset()
    assert a1.value() == 0.0
    p = M.Perplexity()
    p.update(logits[:2], tgt[:2]), p.update(logits[2:], torch.tensor([1, -100]))
    want = torch.nn.functional.cross_entropy(logits[:3], tgt[:3])
    assert p.count() == 3 and p.value() == pytest.approx(math.exp(float(want)), rel=1e-5) and M.Perplexity().value() == float("inf")
    cm = M.ConfusionMatrix(3)
    cm.update(logits, tgt)                                        # predictions 0, 2, 1, 2 against 0, 1, 1, 0
    assert cm.at(0, 0) == 1 and cm.at(2, 1) == 1 and cm.at(1, 1) == 1 and cm.at(2, 0) == 1 and cm.total_samples() == 4
    assert (cm.true_positive(1), cm.false_positive(2), cm.false_negative(0), cm.num_classes(), len(cm.data())) == (1, 2, 1, 3, 9)
    f = M.F1Score(3)
    f.update(logits, tgt)
    assert f.precision(0) == 1.0 and f.recall(0) == 0.5 and f.f1(0) == pytest.approx(2 / 3) and f.f1(2) == 0.0
    assert f.macro_f1() == pytest.approx((2 / 3 + 2 / 3 + 0) / 3) and f.weighted_f1() == pytest.approx(2 / 3)
    assert M.BLEUScore(2).compute(torch.tensor([1, 2, 3, 4]), [1, 2, 3, 4]) == pytest.approx(1.0) and M.BLEUScore().max_n() == 4
    assert M.ROUGELScore().compute([1, 2, 3, 4], [1, 3, 4, 5]) == pytest.approx(0.75)
    mp = M.MeanAveragePrecision()
    assert mp.compute(torch.tensor([0.9, 0.1, 0.8]), torch.tensor([1, 0, 0])) == 1.0 and mp.compute([0.1, 0.9], [1, 0]) == 0.5 and mp.value() == 0.75
    assert S.CosineDecayScheduler is S.CosineDecay and issubclass(S.OneCycleScheduler, S.LRScheduler)
    assert S.ConstantScheduler(0.3).get_lr(99) == 0.3 and S.LambdaScheduler(lambda s: 1.0 / (1 + s)).get_lr(3) == 0.25
    for n in ("LinearDecayScheduler", "ExponentialDecayScheduler", "StepDecayScheduler", "MultiStepDecay", "PolyScheduler", "WarmupScheduler", "CyclicLR",
              "ReduceLROnPlateauScheduler", "SequentialScheduler", "ChainedScheduler"):
        assert issubclass(getattr(S, n), S.Scheduler)


def test_tensor_view_never_copies_and_global_seed_manager(monkeypatch):
    from transformers_fusion_b200.utils import core as C
    from transformers_fusion_b200.utils.random import GlobalSeedManager as G
    base = torch.arange(24.0)
    v = C.TensorView(base, (2, 3, 4))
    assert v.shape() == (2, 3, 4) and v.strides() == [12, 4, 1] and v.rank() == 3 and v.is_contiguous() and v.data_ptr() == base.data_ptr()
    s = v.slice(1, 1, 3)
    assert s.shape() == (2, 2, 4) and s.at(0, 0, 0) == 4.0 and not s.is_contiguous() and s.data_ptr() == base.data_ptr() + 4 * 4
    t = v.transpose(0, 2)
    assert t.shape() == (4, 3, 2) and t.at(3, 2, 1) == 23.0
    with pytest.raises(ValueError):
        t.reshape(24)
    assert v.reshape(6, 4).at(5, 3) == 23.0 and v.narrow(2, 1, 2).at(0, 0, 1) == 2.0
    u = v.unsqueeze(1)
    assert u.shape() == (2, 1, 3, 4) and u.squeeze(1).shape() == (2, 3, 4)
    with pytest.raises(ValueError):
        v.squeeze(0)
    with pytest.raises(IndexError):
        v.slice(0, 1, 3)
    s.data()[0, 0, 0] = -1.0
    assert base[4] == -1.0                                        # a window, not a copy
    c = t.contiguous()
    c[0, 0, 0] = 99.0
    assert base[0] == 0.0 and C.TensorView(base, (2, 2), (1, 2), offset=8).at(1, 1) == 11.0
    monkeypatch.setenv("QUANT_SEED", "1234")
    G.reset()
    assert G.is_deterministic() and G.get_seed() == 1234 and G.next_seed() == 1235 and G.next_seed() == 1236
    monkeypatch.delenv("QUANT_SEED")
    G.reset()
    a = G.get_seed()
    assert not G.is_deterministic() and a != 0 and G.get_seed() == a and G.next_seed() == (a + 1) & 0xFFFFFFFFFFFFFFFF
    monkeypatch.setenv("QUANT_SEED", "0")
    assert not G.is_deterministic()
    G.reset()
