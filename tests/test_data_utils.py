import os

import numpy as np
import pytest
import torch

from transformers_fusion_b200.tokenizer import ByteTokenizer
from transformers_fusion_b200.utils import data as D
from transformers_fusion_b200.utils import random as R
from transformers_fusion_b200.utils import telemetry as T


def test_rng_reproducible_and_distribution(monkeypatch):
    a, b = R.Xoroshiro128Plus(7), R.Xoroshiro128Plus(7)
    assert [a.next_u64() for _ in range(5)] == [b.next_u64() for _ in range(5)] and R.Xoroshiro128Plus(8).next_u64() != R.Xoroshiro128Plus(7).next_u64()
    g = R.Xoroshiro128Plus(1)
    u = [g.uniform() for _ in range(20000)]
    n = [g.normal() for _ in range(20000)]
    assert 0.49 < np.mean(u) < 0.51 and abs(np.mean(n)) < 0.03 and 0.97 < np.std(n) < 1.03 and min(u) >= 0 and max(u) < 1
    assert R.splitmix64(0)[1] == 0xE220A8397B1DCDAF
    assert R.make_seed(42, R.SeedStream.DATA) != R.make_seed(42, R.SeedStream.INIT) and R.make_seed(42, 1, 5) == R.make_seed(42, 1, 5)
    monkeypatch.setenv("QUANT_SEED", "123")
    assert R.resolve_base_seed(0) == 123 and R.resolve_base_seed(9) == 9
    monkeypatch.setenv("QUANT_SEED", "junk")
    assert R.resolve_base_seed(0) == 42


def test_dataset_views_and_split():
    ds = D.InMemoryDataset(list(range(100)))
    ev = ds.filter(lambda x: x % 2 == 0).map(lambda x: x * 10)
    assert len(ev) == 50 and ev[3] == 60
    sh = ds.shuffle(3)
    assert sorted(sh) == list(range(100)) and list(sh) != list(range(100)) and list(ds.shuffle(3)) == list(sh)
    assert len(ds.concat(ev)) == 150 and ds.concat(ev)[100] == 0 and ds.concat(ev)[149] == 980
    tr, va, te = D.split_dataset(ds, (0.8, 0.1, 0.1))
    assert (len(tr), len(va), len(te)) == (80, 10, 10) and sorted(list(tr) + list(va) + list(te)) == list(range(100))
    ch = D.ChunkedDataset(list(range(10)), 4, 3)
    assert len(ch) == 3 and ch[2] == [6, 7, 8, 9]


def test_minhash_and_pipeline(tmp_path):
    dd = D.MinHashDeduper(threshold=0.7)
    base = "the quick brown fox jumps over the lazy dog near the quiet river bank today"
    assert not dd.is_duplicate(base) and dd.is_duplicate(base) and dd.is_duplicate(base.replace("today", "tonight"))
    assert not dd.is_duplicate("completely different words about tensor cores and memory bandwidth on accelerators")
    pre = D.TextPreprocessor(lowercase=True, min_chars=5)
    assert pre("  Ｈello\x00   World  ") == "hello world"
    pipe = D.DataPipeline(ByteTokenizer(), 16, pre, D.MinHashDeduper(threshold=0.7), [lambda s: "spam" not in s])
    rows = pipe.run([base, base, "spam spam spam spam", "hi", "another sufficiently long and distinct document for packing"])
    assert pipe.stats == {"seen": 5, "filtered": 2, "duplicates": 1, "tokens": pipe.stats["tokens"]} and rows.shape[1] == 16 and rows.shape[0] >= 7


def test_loaders(tmp_path):
    D.MmapDataLoader.write_tokens(tmp_path / "t.bin", np.arange(5000) % 1000)
    ml = D.MmapDataLoader(tmp_path / "t.bin", 4, 32)
    x, y = ml.next_batch()
    assert x.shape == (4, 32) and torch.equal(x[:, 1:], y[:, :-1]) and len(ml) == 39
    ml.close()
    (tmp_path / "a.txt").write_text("hello world\n" * 200)
    sl = D.StreamingDataLoader(ByteTokenizer(), [str(tmp_path / "a.txt")], 2, 16)
    batches = list(sl)
    assert len(batches) == (200 * 12) // (2 * 17) and batches[0][0].shape == (2, 16) and torch.equal(batches[0][0][:, 1:], batches[0][1][:, :-1])
    import pyarrow as pa
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"text": ["a", None, "c"], "n": [1, 2, 3]}), tmp_path / "d.parquet")
    pr = D.ParquetReader(tmp_path / "d.parquet")
    assert pr.num_rows() == 3 and list(pr) == ["a", "c"]


def test_generators():
    g = D.DataGenerator(1)
    for line in g.arithmetic(20):
        lhs, rhs = line.split(" = ")
        assert eval(lhs) == int(rhs)
    assert all(s.split(" -> ")[0][::-1] == s.split(" -> ")[1] for s in g.copy_task(5, reverse=True))
    z = g.zipf_tokens(5000, 100)
    assert z.min() >= 0 and z.max() < 100 and (z == 0).mean() > (z == 50).mean()
    assert g.templated(3, ["{a} likes {b}"], {"a": ["x"], "b": ["y", "z"]})[0] in ("x likes y", "x likes z")
    cur = D.CurriculumGenerator(["aaaa", "a", "aaaaaaaa", "aa"], len, start_fraction=0.25)
    assert cur.pool(0.0) == ["a"] and cur.pool(1.0)[-1] == "aaaaaaaa" and set(cur.sample(0.0, 5)) == {"a"}


def test_telemetry(capsys):
    c = T.CacheHitLogger()
    assert [c.log_access(s) for s in (1 << 10, 1 << 22, 1 << 30)] == ["L1", "L2", "HBM"] and abs(sum(c.report().values()) - 1) < 1e-9
    m = T.MemoryTracker()
    m.add("weights", 100), m.add("activations", 50), m.add("offload", 1000)
    assert m.total() == 150 and m.verify_footprint(160) and not m.verify_footprint(400)
    h = T.RoutingHistogram(4)
    h.record(torch.tensor([[0, 1], [2, 3]]))
    assert h.is_balanced() and "expert   0" in h.render()
    h.record([0] * 20)
    assert not h.is_balanced()
    kq = T.KVCacheQuantizer(4, 8)
    assert kq.plan(20) == {"ternary": (0, 8), "q4": (8, 16), "fp": (16, 20)} and kq.tier(0) == "fp" and kq.tier(5) == "q4" and kq.tier(50) == "ternary"
    assert kq.bytes_per_token(20) < 2.0 and kq.bytes_per_token(3) == 2.0
    x = torch.randn(4, 64)
    assert torch.equal(kq.quantize(x, "fp"), x) and (kq.quantize(x, "q4") - x).abs().max() < 0.5 and len(torch.unique(kq.quantize(x, "ternary")[0, :32].abs())) <= 2
    line = T.TelemetryPrinter.print_training_step(3, 2.0, 1e-3, 1234.5, 0.7, m)
    assert line.startswith("Step 3 | loss: 2 | ppl: 7.38906 | lr: 0.001 | tok/s: 1234.5") and "Step 3" in capsys.readouterr().out


def test_reference_dataset_verbs(tmp_path):
    import numpy as np
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    tok = ByteTokenizer()
    (tmp_path / "a.txt").write_text("hello world, this is a text file with enough characters in it")
    (tmp_path / "b.txt").write_text("second file of the directory, also long enough to cut windows")
    ds = D.InMemoryDataset.from_text_file(str(tmp_path / "a.txt"), tok, 8, stride=4, max_samples=5)
    assert ds.size() == 5 and ds.get(1)[0].tolist() == tok.encode("o world,")[:8] and torch.equal(ds.get(0)[0][1:], ds.get(0)[1][:-1])
    assert len(ds.inputs()) == len(ds.targets()) == 5
    both = D.InMemoryDataset.from_directory(str(tmp_path), ".txt", tok, 8)
    assert both.size() == D.InMemoryDataset.from_text_file(str(tmp_path / "a.txt"), tok, 8).size() + \
        D.InMemoryDataset.from_text_file(str(tmp_path / "b.txt"), tok, 8).size()
    np.arange(100, dtype=np.int64).tofile(tmp_path / "t.bin")
    tk = D.InMemoryDataset.from_tokenized_file(str(tmp_path / "t.bin"), 9, max_samples=3)
    assert tk.size() == 3 and tk.get(2)[0].tolist() == list(range(18, 27)) and tk.get(2)[1][-1] == 27
    ds.add_sample(torch.zeros(8), torch.ones(8))
    assert ds.size() == 6
    ds.clear()
    assert ds.size() == 0
    m = D.MapDataset(tk, lambda x, y: (x + 1, y))
    assert m.get(0)[0][0] == 1
    m.set_map_fn(lambda pair: pair[1])
    assert m.get(0).tolist() == list(range(1, 10))
    f = D.FilterDataset(tk, lambda x, y: int(x[0]) >= 9)
    assert f.filtered_indices() == [1, 2] and f.size() == 2
    c = D.ConcatDataset()
    c.add_dataset(tk), c.add_dataset(f)
    assert c.num_datasets() == 2 and c.size() == 5 and c.get(3)[0][0] == 9
    sh = D.ShuffleDataset(D.InMemoryDataset(list(range(20))), seed=1, buffer_size=5)
    p = sh.permutation()
    assert sorted(p) == list(range(20)) and all(i // 5 == v // 5 for i, v in enumerate(p))
    sh.reshuffle()
    assert sh.permutation() != p and sorted(sh.permutation()) == list(range(20))
    ch = D.ChunkedDataset(str(tmp_path / "t.bin"), 10, overlap=5)
    assert ch.num_chunks() == 19 and list(ch.get(1)) == list(range(5, 15))
    ch.set_overlap(0)
    assert ch.num_chunks() == 10
    # token shards: whitespace-separated ids, read through a small buffer
    (tmp_path / "s0.tok").write_text(" ".join(map(str, range(0, 50))))
    (tmp_path / "s1.tok").write_text("\n".join(map(str, range(50, 80))) + "\n")
    st = D.StreamingDataset(str(tmp_path / "s*.tok"), seq_len=8, buffer_size=16)
    assert st.has_next() and st.next_chunk(5) == [0, 1, 2, 3, 4]
    x, y = st.get(0)
    assert x.tolist() == list(range(5, 13)) and y.tolist() == list(range(6, 14))
    assert st.get(1)[0].tolist() == list(range(13, 21))          # windows continue where the last one ended
    rest = st.next_chunk(1000)
    assert rest[0] == 21 and rest[-1] == 79 and not st.has_next() and st.num_chunks() > 0
    st.reset()
    assert st.next_chunk(2) == [0, 1]
    st.shuffle()
    assert sorted(st.next_chunk(1000)) == list(range(80))


def test_text_preprocessor_passes_and_pipeline_stages(tmp_path):
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    p = D.TextPreprocessor()
    p.set_html_stripping(True), p.set_url_removal(True), p.set_email_removal(True), p.set_accent_removal(True), p.set_lowercase(True)
    out = p.process("<p>Visit https://example.com/x?y=1 or mail Bob@Example.org — Café   déjà</p><script>evil()</script>")
    assert out == "visit or mail — cafe deja"
    q = D.TextPreprocessor()
    q.set_pii_removal(True)
    red = q.process("SSN 123-45-6789, card 4111 1111 1111 1111, call +1 (555) 123-4567, host 10.0.0.12, a@b.io")
    assert "123-45-6789" not in red and "4111" not in red and "555" not in red and "10.0.0.12" not in red and "[EMAIL]" in red
    assert "SSN" in red and "call" in red
    q2 = D.TextPreprocessor()
    q2.set_min_length(10), q2.set_max_length(12)
    assert q2.process("short") == "" and q2.process("a much longer sentence") == "a much longe"
    d = D.TextPreprocessor()
    d.set_deduplication(True), d.set_fuzzy_dedup_threshold(0.8)
    texts = ["the quick brown fox jumps over the lazy dog", "the quick brown fox jumps over the lazy dog",
             "the quick brown fox jumps over the lazy dog!", "completely different sentence about kernels"]
    assert d.process_batch(texts) == [texts[0], texts[3]]
    assert d.fuzzy_similarity("abcdef", "abcdef") == 1.0 and d.fuzzy_similarity("abcdef", "uvwxyz") == 0.0
    assert [D.TextPreprocessor.detect_language(t) for t in ("the model is in the loop", "el modelo es de los datos y que",
            "это модель", "这是模型", "これはモデルです", "모델입니다", "12345")] == ["en", "es", "ru", "zh", "ja", "ko", "unknown"]
    outs, langs, lens = d.process_with_metadata(["the cat is in the hat", "  "])
    assert outs == ["the cat is in the hat"] and langs == ["en"] and lens == [21]
    pipe = D.DataPipeline()
    bt = ByteTokenizer()
    pipe.set_tokenizer(bt), pipe.set_seq_length(8), pipe.set_batch_size(2), pipe.set_num_workers(2)
    pipe.add_stage("upper", lambda ts: [t.upper() for t in ts])
    batches = pipe.process_texts(["hello world, twelve", "and another line here"])
    assert batches[0].shape == (2, 8) and bt.decode(batches[0][0].tolist()) == "HELLO WO" and pipe.total_processed() == 2
    pipe.clear_pipeline()
    (tmp_path / "f.txt").write_text("first line of text\n\nsecond line of text\n")
    b2 = pipe.process_file(str(tmp_path / "f.txt"))
    assert bt.decode(b2[0][0].tolist()) == "first li" and pipe.run_stage2(["ab"]) == [bt.encode("ab")]


def test_task_generators_curriculum_and_tokenizer_report(tmp_path):
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    g = D.DataGenerator(3)
    for s in g.generate_arithmetic(20, "+-*"):
        lhs, rhs = s.split(" = ")
        assert eval(lhs) == int(rhs)
    assert all(s.split(" -> ")[0].split(": ")[1] == s.split(" -> ")[1] for s in g.generate_copy_tasks(5, 9))
    assert all(s.split(" -> ")[0].split(": ")[1][::-1] == s.split(" -> ")[1] for s in g.generate_reverse_tasks(5, 9))
    for s in g.generate_sorting_tasks(5, 6):
        a, b = s[6:].split(" -> ")
        assert sorted(map(int, a.split())) == list(map(int, b.split()))
    for s in g.generate_masked_prediction(5, 6):
        a, b = s.split(" -> ")
        assert a.count("[MASK]") == 1 and b in D.DataGenerator._WORDS
    for s in g.generate_next_token_prediction(5, 6):
        xs, nxt = s.split(" -> ")
        xs = list(map(int, xs.split()))
        assert int(nxt) - xs[-1] == xs[1] - xs[0]
    for s in g.generate_pattern_recognition(3, 4):
        a, b = s.split(" -> ")
        assert a.split()[:4] == b.split() and len(a.split()) == 12
    assert all(len(a.split()) == len(b.split()) for a, b in (s.split(" -> ") for s in g.generate_token_recovery(4, 7)))
    assert len(g.generate_random_text(4, 10, 20)) == 4 and len(g.generate_ngram_text(3, 12, 3)[0].split()) == 14
    only_sort = g.generate_mixed(6, [0, 0, 0, 0, 0, 1.0])
    assert all(s.startswith("sort: ") for s in only_sort) and len(g.generate_mixed(7)) == 7
    assert D.DataGenerator(3).generate_copy_tasks(3) == D.DataGenerator(3).generate_copy_tasks(3)
    cur = D.CurriculumGenerator()
    seen = []
    cur.set_progress_fn(lambda name, diff, acc: seen.append((name, diff)))
    cur.add_stage("hard", 2, lambda n: ["h"] * n, max_samples=100, accuracy_threshold=0.8)
    cur.add_stage("easy", 1, lambda n: ["e"] * n, max_samples=5, accuracy_threshold=0.9)
    assert cur.current_stage_name() == "easy" and cur.generate_next_batch(3) == ["e"] * 3
    cur.report_accuracy(0.5)
    assert cur.current_stage_name() == "easy" and seen == [("easy", 1)]
    cur.generate_next_batch(3)                                   # 6 samples: the stage's budget is used up
    assert cur.current_stage_name() == "hard" and cur.current_difficulty() == 2
    cur.report_accuracy(0.95)
    assert cur.is_complete() and cur.generate_next_batch(2) == []
    ev = D.TokenizerEvaluator(ByteTokenizer())
    rep = ev.evaluate("héllo wörld")
    assert rep["total_tokens"] == 13 and rep["corpus_size_bytes"] == 13 and rep["reconstruction_fidelity"] == 1.0
    assert rep["re_encoding_accuracy"] == 1.0 and rep["oov_count"] == 0 and rep["compression_ratio"] == 1.0
    assert ev.character_error_rate("kitten", "sitting") == pytest.approx(3 / 6)
    # memory-mapped loader verbs and the Parquet reader
    D.MmapDataLoader.write_tokens(str(tmp_path / "m.bin"), list(range(64)) * 8 + list(range(500, 756)))
    ml = D.MmapDataLoader(str(tmp_path / "m.bin"), 2, 16)
    x, y = ml.next_batch_with_labels()
    assert x.shape == (2, 16) and ml.has_next() and ml.num_batches() == len(ml)
    assert ml.dedup(window=64) == [1, 2, 3, 4, 5, 6, 7]            # seven repeats of the first 64-token span
    ml.reset(seed=5)
    ml.close()
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"text": ["abc", None, "defgh"]}), str(tmp_path / "d.parquet"))
    r = D.ParquetReader()
    assert not r.open(str(tmp_path / "missing.parquet")) and r.open(str(tmp_path / "d.parquet"))
    assert r.next_batch(4) == list(b"abcd") and r.next_batch(10) == list(b"efgh") and r.next_batch(10) == []
    assert r.rows_read() == 2 and r.total_tokens() == 8
    r.reset()
    assert r.next_batch(2) == list(b"ab")
    r.close()


def test_telemetry_reference_verbs(capsys):
    c = T.CacheHitLogger.instance()
    assert T.CacheHitLogger.instance() is c
    c.reset()
    c.record_sequential(1 << 20, 8, 64)
    c.record_access(1 << 40, 64)
    st = c.stats()
    assert st["total_accesses"] == 9 and st["sequential_reads"] == 7 and st["ram_fetches"] == 2 and st["l1_hits"] == 7
    assert "HBM" in c.print_report()
    m = T.MemoryTracker.instance()
    m.reset()
    m.track_weights("w", 1000), m.track_weights("w", 500), m.track_gradients("g", 2000), m.track_optimizer("o", 2000, 2000)
    m.track_activations("a", 100), m.track_kv_cache(50), m.track_offload("cpu", 7000)
    bd = m.breakdown()
    assert bd["weights_bytes"] == 500 and bd["optimizer_bytes"] == 4000 and bd["total_device_bytes"] == 6650 and bd["total_bytes"] == 13650
    assert m.bpw(1000) == 4.0 and m.verify_bpw(1000, 4.2, 0.1) and not m.verify_bpw(1000, 8.0)
    assert m.update() == 6650 and "bits per weight" in m.print_report(1000, 4.0)
    h = T.RoutingHistogram(3)
    h.record_with_modalities(torch.tensor([[0, 1], [0, 2], [0, 1]]), ["text", "image", "text"])
    e = h.entries()
    assert [x["tokens_routed"] for x in e] == [3, 2, 1] and e[0]["modality_name"] == "text" and e[2]["modality_name"] == "image"
    assert "load-balance loss" in h.print_with_loss(1.5) and "expert" in h.print()
    h.reset()
    assert sum(x["tokens_routed"] for x in h.entries()) == 0
    q = T.KVCacheQuantizer(recent=4, middle=8)
    k, v = torch.randn(20, 2, 32), torch.randn(20, 2, 32)
    k0 = k.clone()
    saved = q.quantize_old_states(k, v, 20)
    assert saved > 0 and torch.equal(k[16:], k0[16:]) and not torch.equal(k[:8], k0[:8]) and k[:8].unique().numel() < 200
    assert q.bytes_saved() == saved and q.compression_ratio() > 1.5 and 0 < q.estimated_quality_loss() < 0.1
    assert torch.equal(q.restore_for_attention(k, 2, 6), k[2:6].float()) and q.config()["quant4_window"] == 8
    T.TelemetryPrinter.routing, T.TelemetryPrinter.kv = h, q
    T.TelemetryPrinter.print_all_header(), T.TelemetryPrinter.print_cache_report(), T.TelemetryPrinter.print_memory_report(1000, 4.0)
    T.TelemetryPrinter.print_routing_report(0.5), T.TelemetryPrinter.print_kv_quant_report(), T.TelemetryPrinter.print_all_footer()
    out = capsys.readouterr().out
    assert "telemetry" in out and "kv cache: saved" in out and "memory:" in out
    T.TelemetryPrinter.routing = T.TelemetryPrinter.kv = None


def test_tokenizer_evaluator_comparison_and_report():
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    from transformers_fusion_b200.utils.data import TokenizerEvaluator
    docs = ["hello world", "second line"]
    reps = TokenizerEvaluator.compare_tokenizers([ByteTokenizer(), ByteTokenizer()], docs)
    assert len(reps) == 2 and reps[0]["tokenizer"] == "ByteTokenizer" and reps[0]["reconstruction_fidelity"] == 1.0
    assert reps[0]["corpus_size_bytes"] == len("hello world\nsecond line")
    text = TokenizerEvaluator.report_string(reps[0])
    assert "compression_ratio" in text and "total_tokens" in text and len(text.splitlines()) == len(reps[0])


def test_streaming_batches_over_token_and_parquet_shards(tmp_path):
    a, b = tmp_path / "a.tok", tmp_path / "b.tok"
    a.write_text(" ".join(str(i) for i in range(0, 20)))
    b.write_text(" ".join(str(i) for i in range(100, 120)))
    ds = D.StreamingDataset([str(a)], seq_len=4)
    ds.add_shard(str(b))
    assert ds.shards_loaded() == 2 and ds.epochs_completed() == 0 and ds.total_tokens() == 0
    x, y = ds.next_batch(3)
    assert x.tolist() == [[0, 1, 2, 3], [5, 6, 7, 8], [10, 11, 12, 13]] and torch.equal(y, x + 1) and ds.total_tokens() == 12
    seen = [x]
    for _ in range(2):
        seen.append(ds.next_batch(3)[0])
    assert seen[1].tolist()[0] == [15, 16, 17, 18] and seen[1].tolist()[1] == [100, 101, 102, 103]
    assert ds.epochs_completed() == 1 and seen[2][-1].tolist() == [0, 1, 2, 3]        # wrapped around to the first shard
    assert D.StreamingDataset([str(a)], seq_len=64).next_batch(1) is None           # less than one window in the shards
    ds.shuffle_shards()
    assert ds.next_batch(1)[0][0, 0].item() in (0, 100)
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    for k in range(2):
        pq.write_table(pa.table({"text": ["abcdefgh" * 4, None, "ijklmnop" * 4][: 3 - k]}), tmp_path / f"s{k}.parquet")
    pds = D.ParquetStreamingDataset(str(tmp_path), vocab_size=64)
    assert pds.shards_loaded() == 2 and pds.size() == 5
    x, y = pds.next_batch(2, 8)
    want = [c % 64 for c in ("abcdefgh" * 4).encode()]
    assert x[0].tolist() == want[:8] and y[0].tolist() == want[1:9] and x[1].tolist() == want[9:17] and int(x.max()) < 64
    n = 0
    while pds.epochs_completed() == 0:
        pds.next_batch(2, 8)
        n += 1
    assert n >= 2 and pds.total_tokens() == (n + 1) * 16
    with pytest.raises(ValueError):
        pds.add_shard(str(a))
    empty = D.ParquetStreamingDataset("", 64, seq_len=8)
    assert empty.shards_loaded() == 0 and empty.next_batch(1) is None
    empty.add_shard(str(tmp_path / "s1.parquet"))
    assert empty.next_batch(1)[0].shape == (1, 8)
