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
        c.sendall(P.ws_encode_frame(b"", 8, mask=b"abcd"))
        c.close()
        bad = socket.create_connection(("127.0.0.1", port))
        bad.sendall(b"GET / HTTP/1.1\r\nHost: x\r\n\r\n")
        assert b"400" in bad.recv(1024)
        bad.close()
    finally:
        ws.stop()


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
