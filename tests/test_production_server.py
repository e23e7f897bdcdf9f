import base64
import json
import os
import socket
import struct
import time

import pytest
import torch

from transformers_fusion_b200.inference.engine import EngineConfig, InferenceEngine
from transformers_fusion_b200.inference.sampler import SamplerConfig
from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.server import production as P
from transformers_fusion_b200.tokenizer import ByteTokenizer


def engine():
    cfg = TransformerConfig(vocab_size=259, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=64)
    m = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0)
    return m, InferenceEngine(m, ByteTokenizer(), EngineConfig(num_pages=64))


def test_latency_histogram():
    h = P.LatencyHistogram()
    for v in range(1, 101):
        h.record(float(v))
    s = h.summary()
    assert s["count"] == 100 and s["p50_ms"] in (50.0, 51.0) and s["p95_ms"] in (95.0, 96.0) and s["p99_ms"] in (99.0, 100.0)


def test_model_server_priorities_and_metrics():
    m, eng = engine()
    ref = eng.generate_batch([[5, 6, 7]], 6, SamplerConfig(0.0))[0]
    ms = P.ModelServer(eng).start()
    try:
        streamed = []
        t1 = ms.submit([5, 6, 7], 6, SamplerConfig(0.0), priority=1, on_token=streamed.append)
        t2 = ms.submit([9, 9], 4, SamplerConfig(0.0), priority=5)
        assert t1.done.wait(30) and t2.done.wait(30)
        assert t1.tokens == ref == streamed and len(t2.tokens) <= 4
        assert ms.generate([5, 6, 7], 6, SamplerConfig(0.0)) == ref
        met = json.loads(ms.metrics_json())
        assert met["requests_total"] == 3 and met["tokens_generated"] >= 12 and met["latency"]["count"] == 3 and met["ttft"]["count"] == 3
        assert json.loads(ms.health_json())["status"] == "ok"
        small = P.ModelServer(eng, max_queue=0)
        t = small.submit([1], 1)
        assert t.error == "queue full"
    finally:
        ms.stop()
    assert json.loads(ms.health_json())["status"] == "stopped"


def test_websocket_roundtrip():
    assert P.websocket_accept_key("dGhlIHNhbXBsZSBub25jZQ==") == "s3pPLMBiTxaQ9kYGzzhZRbK+xOo="      # RFC 6455 example
    for n in (5, 300, 70000):
        fr = P.ws_encode_frame(b"x" * n, mask=b"\x01\x02\x03\x04")
        op, payload, used = P.ws_decode_frame(fr)
        assert op == 1 and payload == b"x" * n and used == len(fr) and P.ws_decode_frame(fr[:-1]) is None

    def on_msg(text, send):
        for ch in text:
            send(ch.upper())
    ws = P.WebSocketHandler(0, on_msg)
    port = ws.start()
    try:
        c = socket.create_connection(("127.0.0.1", port))
        key = base64.b64encode(os.urandom(16)).decode()
        c.sendall((f"GET / HTTP/1.1\r\nHost: x\r\nUpgrade: websocket\r\nConnection: Upgrade\r\nSec-WebSocket-Key: {key}\r\n"
                   "Sec-WebSocket-Version: 13\r\n\r\n").encode())
        resp = b""
        while b"\r\n\r\n" not in resp:
            resp += c.recv(1024)
        assert b"101 Switching Protocols" in resp and P.websocket_accept_key(key).encode() in resp
        c.sendall(P.ws_encode_frame(b"abc", mask=b"abcd"))
        buf, got = resp.split(b"\r\n\r\n", 1)[1], []
        while len(got) < 3:
            fr = P.ws_decode_frame(buf)
            if fr is None:
                buf += c.recv(1024)
                continue
            got.append(fr[1].decode())
            buf = buf[fr[2]:]
        assert got == ["A", "B", "C"]
        assert ws.is_running() and ws.broadcast("tok") == 1
        while True:
            fr = P.ws_decode_frame(buf)
            if fr is not None:
                break
            buf += c.recv(1024)
        assert fr[1] == b"tok"
        buf = buf[fr[2]:]
        c.sendall(P.ws_encode_frame(b"", 8, mask=b"abcd"))
        c.close()
        bad = socket.create_connection(("127.0.0.1", port))
        bad.sendall(b"GET / HTTP/1.1\r\nHost: x\r\n\r\n")
        assert b"400" in bad.recv(1024)
        bad.close()
    finally:
        ws.stop()
    assert not ws.is_running()


def test_plugins_and_zoo(tmp_path):
    p = tmp_path / "plug.py"
    p.write_text("def plugin_init(ctx):\n    return ctx + 1\n\ndef hello(x):\n    return 'v1:' + x\n")
    pm = P.PluginManager()
    name = pm.load(str(p), 41)
    assert pm.plugins[name]["result"] == 42 and pm.call(name, "hello", "a") == "v1:a" and pm.reload_changed() == []
    time.sleep(0.02)
    p.write_text("def plugin_init(ctx):\n    return ctx\n\ndef hello(x):\n    return 'v2:' + x\n")
    os.utime(p, (time.time() + 2, time.time() + 2))
    assert pm.reload_changed() == [name] and pm.call(name, "hello", "a") == "v2:a"
    pm.unload(name)
    assert pm.names() == []
    from transformers_fusion_b200.quant import codec
    m, _ = engine()
    codec.save_model(m, tmp_path / "tiny.quant")
    zoo = P.ModelZoo()
    assert zoo.scan(str(tmp_path)) == ["tiny"]
    m2 = zoo.get("tiny")
    assert zoo.get("tiny") is m2 and m2.cfg.hidden_size == 32
    zoo.unload("tiny")
    assert "tiny" not in zoo.loaded


def test_model_server_load_unload_and_named_helpers(tmp_path):
    from transformers_fusion_b200.quant import codec
    from transformers_fusion_b200.utils.logging import AppConfig, Logger
    m, eng = engine()
    other = DenseModel(m.cfg, device="cpu", dtype=torch.float32, seed=9)
    codec.save_model(other, str(tmp_path / "other.quant"))
    want = InferenceEngine(other, ByteTokenizer(), EngineConfig(num_pages=64)).generate_batch([[5, 6, 7]], 5, SamplerConfig(0.0))[0]
    ms = P.ModelServer(eng).start()
    try:
        assert ms.is_running() and ms.is_model_loaded()
        ms.set_batch_size(3), ms.set_queue_wait_ms(2)
        assert eng.cfg.max_batch == 3 and ms.queue_wait_s == 0.002
        first = ms.generate([5, 6, 7], 5, SamplerConfig(0.0))
        assert not ms.load_model(str(tmp_path / "missing.quant")) and ms.is_model_loaded()      # a bad path changes nothing
        assert ms.load_model(str(tmp_path / "other.quant"))
        assert ms.generate([5, 6, 7], 5, SamplerConfig(0.0)) == want != first
        ms.unload_model()
        assert not ms.is_model_loaded() and ms.submit([1], 1).error == "no model is loaded"
        assert ms.metrics.avg_latency_ms() > 0 and ms.metrics.requests_per_sec() > 0
        h = ms.metrics.latency
        assert h.p50() <= h.p95() <= h.p99()
    finally:
        ms.stop()
    assert not ms.is_running()
    # process-wide logger with a file, numeric levels
    log = Logger.instance()
    assert Logger.instance() is log
    old_stream, log.stream = log.stream, None
    log.set_file(str(tmp_path / "app.log"))
    log.set_level(2)
    log.log(1, "quiet"), log.log(Logger.ERROR, "loud"), log.log(3, "numeric")
    log.set_file(None)
    log.stream = old_stream
    log.set_level("info")
    text = (tmp_path / "app.log").read_text()
    assert "quiet" not in text and "[ERROR] loud" in text and "[ERROR] numeric" in text
    cfg = AppConfig()
    cfg.set("server.port", "8080"), cfg.set("server.rate", "2.5"), cfg.set("server.debug", "true"), cfg.set("name", "tfb")
    assert cfg.get_int("server.port") == 8080 and cfg.get_float("server.rate") == 2.5 and cfg.get("server.debug") is True
    assert cfg.get_string("name") == "tfb" and cfg.get_string("server.debug") == "true" and cfg.get_int("nope", 7) == 7
    assert cfg.get_int("name", 3) == 3 and json.loads(cfg.to_json())["server"]["port"] == 8080
    # plugin hooks: objects registered directly and Python files
    (tmp_path / "plug.py").write_text("seen = []\ndef on_generate_start(p): seen.append(('start', p))\ndef on_token_generated(t): seen.append(('tok', t))\n")
    pm = P.PluginManager()
    name = pm.load(str(tmp_path / "plug.py"))

    class Direct:
        def __init__(self):
            self.ends = []

        def name(self): return "direct"
        def on_generate_end(self, out): self.ends.append(out)
        def on_token_generated(self, t): raise RuntimeError("faulty plugin")
    d = Direct()
    pm.register_plugin(d)
    pm.on_generate_start("hi"), pm.on_token_generated(5), pm.on_generate_end("done")
    assert pm.direct_plugin_count() == 1 and d.ends == ["done"]
    assert pm.plugins[name]["module"].seen == [("start", "hi"), ("tok", 5)]
    (tmp_path / "plug.py").write_text("seen = ['fresh']\n")
    assert pm.hot_reload(str(tmp_path / "plug.py")) and pm.plugins[name]["module"].seen == ["fresh"]
    assert not pm.hot_reload(str(tmp_path / "missing.py"))
    pm.unload_all()
    assert pm.names() == [] and pm.direct_plugin_count() == 0
    zoo = P.ModelZoo()
    zoo.scan(str(tmp_path))
    info = zoo.list_models()
    assert info[0]["name"] == "other" and info[0]["params"] == sum(p.numel() for p in other.parameters()) and info[0]["format"] == "Q_32"
    assert zoo.load("other") is zoo.get("other")
