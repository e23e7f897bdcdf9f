import json

import pytest

from transformers_fusion_b200.utils import gle, metrics
from transformers_fusion_b200.utils.logging import AppConfig, EventWriter, Logger, WandBLogger, crc32c, read_event_scalars
from transformers_fusion_b200.utils.profiling import DeviceTimer, MemoryTracker, benchmark_operation


def test_metrics():
    assert metrics.accuracy([1, 2, 3], [1, 0, 3]) == pytest.approx(2 / 3)
    assert metrics.perplexity(0.0) == 1.0
    assert metrics.bleu("the cat sat on the mat".split(), ["the cat sat on the mat".split()]) == pytest.approx(1.0)
    assert 0 < metrics.bleu("the cat sat".split(), ["the cat sat on the mat".split()]) < 0.6
    assert metrics.bleu("dog".split(), ["the cat".split()]) == 0.0
    r = metrics.rouge_n("a b c d".split(), "a b x d".split(), 1)
    assert r["precision"] == 0.75 and r["recall"] == 0.75
    assert metrics.rouge_l("a b c d".split(), "a c d".split())["recall"] == 1.0
    assert metrics.f1_score([1, 1, 0, 0], [1, 0, 1, 0]) == 0.5
    cm = metrics.confusion_matrix([0, 1, 1], [0, 1, 0], 2)
    assert cm.tolist() == [[1, 1], [0, 1]]
    import torch
    rep = metrics.eval_classification(torch.tensor([[2.0, 0], [0, 2.0], [2.0, 0]]), [0, 1, 1])
    assert rep.accuracy == pytest.approx(2 / 3) and 0 < rep.f1_score < 1


def test_event_writer_and_wandb(tmp_path):
    assert crc32c(b"123456789") == 0xE3069283
    w = EventWriter(str(tmp_path / "tb"))
    for s in range(3):
        w.write_scalar("train/loss", 3.0 - s, s)
    w.close()
    got = read_event_scalars(w.path)
    assert [(s, t) for s, t, _ in got] == [(0, "train/loss"), (1, "train/loss"), (2, "train/loss")]
    assert [v for _, _, v in got] == [3.0, 2.0, 1.0]
    wb = WandBLogger("proj", "r1", root=str(tmp_path))
    wb.log("loss", 1.5, 7)
    wb.close()
    row = json.loads(open(wb.path).read().strip())
    assert row["loss"] == 1.5 and row["_step"] == 7


def test_logger_and_config(tmp_path):
    lg = Logger("warn", str(tmp_path / "log.txt"), stream=None)
    lg.info("hidden")
    lg.error("shown")
    lg.close()
    txt = open(tmp_path / "log.txt").read()
    assert "shown" in txt and "hidden" not in txt and "[ERROR]" in txt
    c = AppConfig(str(tmp_path / "c.json"))
    c.set("server.port", 8080)
    c.set("server.auth.token", "x")
    c.save()
    c2 = AppConfig(str(tmp_path / "c.json"))
    assert c2.get("server.port") == 8080 and c2.get("server.missing", 5) == 5
    assert c2.validate({"server.port": int, "server.auth.token": str}) == []
    assert c2.validate({"server.port": str, "model.path": str}) == ["server.port: expected str, got int", "model.path: missing"]


def test_gle_chain(tmp_path):
    p = str(tmp_path / "t.jsonl")
    w = gle.TelemetryWriter(p)
    h1 = w.append(gle.Event(run_id="r", type="RUN_STARTED", actor="driver"))
    w.append(gle.Event(run_id="r", type="TEST_RESULT", verdict="PASS", evidence="log.txt", numbers={"n": 3}))
    w.close()
    w = gle.TelemetryWriter(p)                        # reopening continues the chain
    w.append(gle.Event(run_id="r", type="RUN_ENDED"))
    w.close()
    r = gle.TelemetryReader(p)
    assert r.report().chain_valid and r.report().events_parsed == 3 and r.events[0].hash == h1 and r.events[1].prev_hash == h1
    assert "chain: VALID" in gle.report(p) and "TEST_RESULT: 1" in gle.report(p) and "PASS=1" in gle.report(p)
    lines = open(p).read().split("\n")
    open(p, "w").write("\n".join([lines[0], lines[1].replace('"PASS"', '"FAIL"'), lines[2]]) + '\n{"partial')
    rep = gle.TelemetryReader(p).report()
    assert not rep.chain_valid and rep.first_bad_line == 2 and rep.truncated_tail
    assert gle.fnv1a64(b"") == 0xCBF29CE484222325 and gle.fnv1a64(b"a") == 0xAF63DC4C8601EC8C


def test_profiling_helpers():
    t = DeviceTimer()
    with t("phase"):
        sum(range(1000))
    s = t.summary()
    assert s["phase"]["calls"] == 1 and s["phase"]["total_ms"] >= 0
    perf = benchmark_operation(lambda: sum(range(100)), iters=3, warmup=1, nbytes=1000)
    assert perf.ms > 0 and perf.gbs > 0
    m = MemoryTracker()
    m.alloc("a", 100)
    m.alloc("b", 50)
    m.free("a")
    assert m.report()["current"] == 50 and m.report()["peak"] == 150
