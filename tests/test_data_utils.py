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
