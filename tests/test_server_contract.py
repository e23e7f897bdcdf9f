"""OpenAI wire contract of the native HTTP server: exact helper bytes, hardening defaults, and a live
server on an ephemeral port driven through raw sockets (limits, auth, rate limit, routes, SSE)."""
import json
import socket

import pytest

from transformers_fusion_b200.server import HTTPServer


def test_error_shape_and_sse_frames():
    j = json.loads(HTTPServer.openai_error_json("bad request", "invalid_request_error", "invalid_json"))
    assert j == {"error": {"message": "bad request", "type": "invalid_request_error", "code": "invalid_json"}}
    assert json.loads(HTTPServer.openai_error_json("x"))["error"]["type"] == "invalid_request_error"
    assert HTTPServer.sse_data_frame('{"a":1}') == 'data: {"a":1}\n\n'
    assert HTTPServer.sse_done_frame() == "data: [DONE]\n\n"


def test_hardening_defaults_and_setters():
    s = HTTPServer(0)
    assert s.auth_token() == "" and s.max_header_bytes() == 64 * 1024 and s.max_concurrent() == 0
    assert not s.is_running() and s.current_requests() == 0
    s.set_auth_token("sekret"); s.set_max_header_bytes(8192); s.set_max_concurrent(8)
    assert s.auth_token() == "sekret" and s.max_header_bytes() == 8192 and s.max_concurrent() == 8
    s.set_max_header_bytes(-1); s.set_max_concurrent(-3)
    assert s.max_header_bytes() == 64 * 1024 and s.max_concurrent() == 0


def _raw(port, payload: bytes, read_all=True):
    c = socket.create_connection(("127.0.0.1", port), timeout=10)
    c.sendall(payload)
    data = b""
    while True:
        b = c.recv(65536)
        if not b:
            break
        data += b
    c.close()
    head, _, body = data.partition(b"\r\n\r\n")
    return int(head.split()[1]), head.decode(), body


def _post(port, path, obj, headers=""):
    body = json.dumps(obj).encode()
    req = f"POST {path} HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: {len(body)}\r\n{headers}\r\n".encode() + body
    return _raw(port, req)


@pytest.fixture()
def server():
    s = HTTPServer(0)
    s.set_model_name("unit-model")
    s.set_generate_callback(lambda prompt, max_tokens, t, p, k, stream: ["echo:", prompt[:8], "!"][: max(1, min(3, max_tokens))])
    s.set_embeddings_callback(lambda text: [float(len(text)), 1.0, 2.0])
    assert s.start()
    yield s
    s.stop()


def test_live_routes(server):
    port = server.port
    code, _, body = _raw(port, b"GET /health HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 200 and json.loads(body)["status"] == "ok"
    code, _, body = _raw(port, b"GET /v1/models HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 200 and json.loads(body)["data"][0]["id"] == "unit-model"
    code, head, body = _post(port, "/v1/completions", {"prompt": "hello world", "max_tokens": 3})
    j = json.loads(body)
    assert code == 200 and j["object"] == "text_completion" and j["choices"][0]["text"] == "echo:hello wo!"
    assert j["usage"]["completion_tokens"] == 3 and "Access-Control-Allow-Origin" in head
    code, _, body = _post(port, "/v1/completions", {"prompt": ["a", "b"], "max_tokens": 9999})
    assert code == 200 and len(json.loads(body)["choices"]) == 2
    code, _, body = _post(port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2})
    j = json.loads(body)
    assert code == 200 and j["choices"][0]["message"]["role"] == "assistant"
    code, _, body = _post(port, "/v1/embeddings", {"input": ["abc", "de"]})
    j = json.loads(body)
    assert code == 200 and j["data"][1]["embedding"][0] == 2.0
    code, _, body = _post(port, "/v1/embeddings", {"input": ["x"] * 257})
    assert code == 400
    code, _, body = _raw(port, b"GET /nope HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 404 and "error" in json.loads(body)
    code, _, _ = _raw(port, b"OPTIONS /v1/completions HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 204
    code, _, body = _raw(port, b"GET /metrics HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 200 and b"tfb_requests_total" in body


def test_live_streaming(server):
    code, head, body = _post(server.port, "/v1/chat/completions",
                             {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3, "stream": True})
    assert code == 200 and "text/event-stream" in head
    frames = [f for f in body.decode().split("\n\n") if f]
    assert all(f.startswith("data: ") for f in frames) and frames[-1] == "data: [DONE]"
    first = json.loads(frames[0][6:])
    assert first["choices"][0]["delta"] == {"role": "assistant"}
    text = "".join(json.loads(f[6:])["choices"][0]["delta"].get("content", "") for f in frames[1:-1])
    assert text.startswith("echo:")


def test_live_limits_and_auth(server):
    port = server.port
    code, _, _ = _raw(port, b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nTransfer-Encoding: chunked\r\nContent-Type: application/json\r\n\r\n0\r\n\r\n")
    assert code == 501
    code, _, _ = _raw(port, b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: text/plain\r\nContent-Length: 2\r\n\r\n{}")
    assert code == 415
    code, _, _ = _raw(port, b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: 99999999\r\n\r\n")
    assert code == 413
    code, _, _ = _raw(port, b"GET /" + b"a" * 9000 + b" HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 414
    code, _, _ = _raw(port, b"GET /health HTTP/1.1\r\nHost: x\r\nX-Big: " + b"b" * 70000 + b"\r\n\r\n")
    assert code == 431
    code, _, body = _post(port, "/v1/completions", {"prompt": 5})
    assert code == 400 and json.loads(body)["error"]["type"] == "invalid_request_error"
    code, _, _ = _raw(port, b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: 5\r\n\r\n{bad}")
    assert code == 400
    server.set_auth_token("tok")
    code, _, _ = _post(port, "/v1/completions", {"prompt": "x"})
    assert code == 401
    code, _, _ = _post(port, "/v1/completions", {"prompt": "x"}, "Authorization: Bearer tok\r\n")
    assert code == 200
    code, _, _ = _raw(port, b"GET /health HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 200   # auth only guards /v1/*
    server.set_auth_token("")
    server.set_rate_limit(0.001, 2)
    codes = [_raw(port, b"GET /health HTTP/1.1\r\nHost: x\r\n\r\n")[0] for _ in range(4)]
    assert codes[:2] == [200, 200] and 429 in codes[2:]


def test_model_load_and_unload_routes(server):
    port = server.port
    code, _, body = _post(port, "/v1/models/load", {"path": "/models/a.quant"})
    assert code == 503 and json.loads(body)["error"]["code"] == "no_load_callback"
    seen = []
    server.set_load_model_callback(lambda path: seen.append(("load", path)) or path.endswith(".quant"))
    server.set_unload_model_callback(lambda: seen.append(("unload",)))
    code, _, body = _post(port, "/v1/models/unload", {})
    assert code == 200 and json.loads(body)["status"] == "unloaded"
    code, _, body = _raw(port, b"GET /v1/models HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 200 and json.loads(body)["data"] == []
    code, _, body = _post(port, "/v1/completions", {"prompt": "hi", "max_tokens": 1})
    assert code == 503 and json.loads(body)["error"]["code"] == "model_not_loaded"
    code, _, body = _post(port, "/v1/models/load", {"path": "/models/b.bin"})
    assert code == 500 and json.loads(body)["error"]["code"] == "load_failed"
    code, _, body = _post(port, "/v1/models/load", {"name": "x"})
    assert code == 400
    code, _, body = _post(port, "/v1/models/load", {"path": "/models/a.quant", "name": "second-model"})
    assert code == 200 and json.loads(body) == {"status": "loaded", "model": "second-model", "path": "/models/a.quant"}
    code, _, body = _raw(port, b"GET /v1/models HTTP/1.1\r\nHost: x\r\n\r\n")
    assert json.loads(body)["data"][0]["id"] == "second-model"
    code, _, body = _post(port, "/v1/completions", {"prompt": "hi", "max_tokens": 1})
    assert code == 200 and json.loads(body)["model"] == "second-model"
    assert seen == [("unload",), ("load", "/models/b.bin"), ("load", "/models/a.quant")]
    code, _, _ = _raw(port, b"GET /v1/models/load HTTP/1.1\r\nHost: x\r\n\r\n")
    assert code == 405
    assert server.model_name() == "second-model" and server.total_requests() >= 10 and server.total_errors() >= 4
    assert server.total_tokens() >= 1
