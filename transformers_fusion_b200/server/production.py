"""Serving runtime around the inference engine: ``ModelServer`` (priority queue in front of the continuous-batching loop,
latency histograms, health / metrics JSON), ``ModelHTTPServer`` (the native HTTP front end wired to it),
``WebSocketHandler`` (RFC 6455 server: SHA-1 / base64 handshake, text frames, token streaming), ``PluginManager``
(shared-library and Python plugins with hot reload) and ``ModelZoo`` (named model registry with lazy loading).

Reference counterparts: include/quant/production.h:21-362 (ServerMetrics, LatencyHistogram, ModelServer, ModelHTTPServer,
WebSocketHandler, PluginManager, ModelZoo), src/server/production_core.cpp, production_api.cpp, production_gen.cpp."""
from __future__ import annotations

import base64
import bisect
import ctypes
import hashlib
import importlib.util
import json
import os
import socket
import struct
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


class LatencyHistogram:
    def __init__(self, max_samples=65536):
        self.samples: List[float] = []
        self.max = max_samples
        self.lock = threading.Lock()
        self.count, self.total = 0, 0.0

    def record(self, ms: float):
        with self.lock:
            self.count += 1
            self.total += ms
            bisect.insort(self.samples, ms)
            if len(self.samples) > self.max:
                del self.samples[:: 2]               # keep every other sample: the quantiles stay representative

    def percentile(self, p: float) -> float:
        with self.lock:
            if not self.samples:
                return 0.0
            return self.samples[min(len(self.samples) - 1, int(p / 100.0 * len(self.samples)))]

    def p50(self) -> float: return self.percentile(50.0)
    def p95(self) -> float: return self.percentile(95.0)
    def p99(self) -> float: return self.percentile(99.0)

    def summary(self):
        return {"count": self.count, "mean_ms": self.total / max(1, self.count), "p50_ms": self.percentile(50),
                "p95_ms": self.percentile(95), "p99_ms": self.percentile(99)}


@dataclass
class ServerMetrics:
    requests_total: int = 0
    requests_failed: int = 0
    tokens_generated: int = 0
    queue_depth: int = 0
    active: int = 0
    started_at: float = field(default_factory=time.time)
    latency: LatencyHistogram = field(default_factory=LatencyHistogram)
    ttft: LatencyHistogram = field(default_factory=LatencyHistogram)

    def avg_latency_ms(self) -> float:
        return self.latency.total / max(1, self.latency.count)

    def requests_per_sec(self) -> float:
        return self.requests_total / max(1e-9, time.time() - self.started_at)

    def to_json(self) -> str:
        up = time.time() - self.started_at
        return json.dumps({"requests_total": self.requests_total, "requests_failed": self.requests_failed,
                           "tokens_generated": self.tokens_generated, "queue_depth": self.queue_depth, "active": self.active,
                           "uptime_s": round(up, 3), "tokens_per_sec": self.tokens_generated / max(up, 1e-9),
                           "latency": self.latency.summary(), "ttft": self.ttft.summary()})


class _Ticket:
    def __init__(self, prompt_ids, max_tokens, sampling, priority, on_token):
        self.prompt_ids, self.max_tokens, self.sampling, self.priority, self.on_token = prompt_ids, max_tokens, sampling, priority, on_token
        self.done = threading.Event()
        self.tokens: List[int] = []
        self.error: Optional[str] = None
        self.t_submit = time.perf_counter()
        self.t_first = 0.0


class ModelServer:
    """One engine loop thread; ``submit`` queues a request (higher priority first, FIFO within a priority) and returns a
    ticket; the loop admits tickets into the engine's continuous batch and steps it."""

    def __init__(self, engine, max_queue: int = 1024):
        self.engine, self.max_queue = engine, max_queue
        self.metrics = ServerMetrics()
        self.cv = threading.Condition()
        self.pending: List[_Ticket] = []
        self.inflight: Dict[int, _Ticket] = {}
        self.running = False
        self.thread: Optional[threading.Thread] = None

    def start(self):
        self.running = True
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()
        return self

    def stop(self):
        self.running = False
        with self.cv:
            self.cv.notify_all()
        if self.thread:
            self.thread.join(timeout=5)

    def is_running(self) -> bool:
        return self.running and self.thread is not None and self.thread.is_alive()

    def is_model_loaded(self) -> bool:
        return self.engine is not None

    def set_batch_size(self, n: int):
        """Upper bound on the sequences the engine decodes together (takes effect for requests admitted from now on)."""
        if self.engine is not None:
            self.engine.cfg.max_batch = max(1, int(n))

    def set_queue_wait_ms(self, ms: int):
        """How long the loop sleeps when it has nothing to do before it looks at the queue again."""
        self.queue_wait_s = max(0.0, ms / 1e3)

    def unload_model(self):
        """Stop admitting work, wait for what is in flight and drop the engine; queued tickets fail with "no model"."""
        with self.cv:
            while self.inflight:
                self.cv.wait(0.05)
            for t in self.pending:
                t.error = "no model is loaded"
                t.done.set()
            self.pending, self.engine = [], None
            self.metrics.queue_depth = 0

    def load_model(self, path: str, tokenizer=None, engine_cfg=None) -> bool:
        """Build an engine for the checkpoint at ``path`` and serve from it (the previous engine is drained first)."""
        try:
            from ..inference.engine import EngineConfig, InferenceEngine
            from ..quant import codec
            import torch
            old = self.engine
            dev = old.device if old is not None else ("cuda" if torch.cuda.is_available() else "cpu")
            model = codec.load_model(path, device=dev, dtype=torch.bfloat16 if str(dev).startswith("cuda") else torch.float32)
            eng = InferenceEngine(model, tokenizer or (old.tok if old is not None else None), engine_cfg or (old.cfg if old is not None else EngineConfig()))
        except Exception as e:
            self.last_error = str(e)
            return False
        if self.engine is not None:
            self.unload_model()
        with self.cv:
            self.engine = eng
            self.cv.notify_all()
        return True

    def submit(self, prompt_ids, max_tokens=64, sampling=None, priority=0, on_token=None) -> _Ticket:
        t = _Ticket(list(prompt_ids), max_tokens, sampling, priority, on_token)
        with self.cv:
            if self.engine is None:
                t.error = "no model is loaded"
                t.done.set()
                self.metrics.requests_failed += 1
                return t
            if len(self.pending) >= self.max_queue:
                t.error = "queue full"
                t.done.set()
                self.metrics.requests_failed += 1
                return t
            self.pending.append(t)
            self.pending.sort(key=lambda x: (-x.priority, x.t_submit))
            self.metrics.queue_depth = len(self.pending)
            self.cv.notify_all()
        return t

    def generate(self, prompt_ids, max_tokens=64, sampling=None, priority=0, timeout_s=600.0) -> List[int]:
        t = self.submit(prompt_ids, max_tokens, sampling, priority)
        if not t.done.wait(timeout_s):
            raise TimeoutError("generation timed out")
        if t.error:
            raise RuntimeError(t.error)
        return t.tokens

    def _loop(self):
        while self.running:
            with self.cv:
                eng = self.engine
                while self.running and (eng is None or (not self.pending and not eng.has_pending())):
                    self.cv.wait(getattr(self, "queue_wait_s", 0.05) or 0.001)
                    eng = self.engine
                if not self.running:
                    return
                batch, self.pending = self.pending, []
                self.metrics.queue_depth = 0
            for t in batch:
                def cb(tok, t=t):
                    if not t.tokens:
                        t.t_first = time.perf_counter()
                        self.metrics.ttft.record((t.t_first - t.t_submit) * 1e3)
                    t.tokens.append(tok)
                    if t.on_token:
                        t.on_token(tok)
                try:
                    r = eng.add_request(t.prompt_ids[-(eng.max_len - 2):] or [0], t.max_tokens, t.sampling, priority=t.priority, on_token=cb)
                    self.inflight[r.id] = t
                    self.metrics.requests_total += 1
                except Exception as e:                     # a bad request must not take the loop down
                    t.error = str(e)
                    t.done.set()
                    self.metrics.requests_failed += 1
            try:
                finished = eng.step() if eng.has_pending() else []
            except Exception as e:
                for t in self.inflight.values():
                    t.error = str(e)
                    t.done.set()
                self.metrics.requests_failed += len(self.inflight)
                self.inflight.clear()
                continue
            for r in finished:
                t = self.inflight.pop(r.id, None)
                if t is not None:
                    self.metrics.tokens_generated += len(t.tokens)
                    self.metrics.latency.record((time.perf_counter() - t.t_submit) * 1e3)
                    t.done.set()
            self.metrics.active = len(self.inflight)
            if finished:
                with self.cv:
                    self.cv.notify_all()                   # a model swap may be waiting for the engine to drain

    def health_json(self) -> str:
        return json.dumps({"status": "ok" if self.running else "stopped", "queue_depth": self.metrics.queue_depth,
                           "active": self.metrics.active})

    def metrics_json(self) -> str:
        return self.metrics.to_json()


class ModelHTTPServer:
    """OpenAI-compatible HTTP endpoint (native front end) in front of a ``ModelServer``."""

    def __init__(self, model_server: ModelServer, tokenizer, port=8080, model_name="model"):
        from . import HTTPServer
        self.ms, self.tok = model_server, tokenizer
        self.http = HTTPServer(port)
        self.http.set_model_name(model_name)
        self.http.set_generate_callback(self._generate)

    def _generate(self, prompt, max_tokens, temperature, top_p, top_k, stream):
        from ..inference.sampler import SamplerConfig
        ids = self.tok.encode(prompt)
        out = self.ms.generate(ids, max_tokens, SamplerConfig(temperature, top_k, top_p))
        eos = getattr(self.tok, "eos_id", -1)
        yield self.tok.decode([t for t in out if t != eos])

    def start(self):
        self.ms.start()
        return self.http.start()

    def stop(self):
        self.http.stop()
        self.ms.stop()

    def is_running(self) -> bool: return self.http.is_running()
    def set_thread_pool_size(self, n: int): self.http.set_thread_pool_size(n)
    def set_timeout_seconds(self, s: int): self.http.set_timeout_seconds(s)
    def set_max_body_size(self, n: int): self.http.set_max_body_size(n)

    @property
    def port(self):
        return self.http.port


# ================================================================================================ WebSocket
_WS_GUID = "258EAFA5-E914-47DA-95CA-C5AB0DC85B11"


def websocket_accept_key(client_key: str) -> str:
    return base64.b64encode(hashlib.sha1((client_key + _WS_GUID).encode()).digest()).decode()


def ws_encode_frame(payload: bytes, opcode=1, mask: Optional[bytes] = None) -> bytes:
    n = len(payload)
    hdr = bytes([0x80 | opcode])
    mbit = 0x80 if mask else 0
    if n < 126:
        hdr += bytes([mbit | n])
    elif n < 65536:
        hdr += bytes([mbit | 126]) + struct.pack(">H", n)
    else:
        hdr += bytes([mbit | 127]) + struct.pack(">Q", n)
    if mask:
        payload = bytes(b ^ mask[i & 3] for i, b in enumerate(payload))
        hdr += mask
    return hdr + payload


def ws_decode_frame(buf: bytes):
    """(opcode, payload, bytes consumed) or None when ``buf`` does not hold a whole frame yet."""
    if len(buf) < 2:
        return None
    op, n = buf[0] & 0x0F, buf[1] & 0x7F
    masked = bool(buf[1] & 0x80)
    o = 2
    if n == 126:
        if len(buf) < 4:
            return None
        n, o = struct.unpack(">H", buf[2:4])[0], 4
    elif n == 127:
        if len(buf) < 10:
            return None
        n, o = struct.unpack(">Q", buf[2:10])[0], 10
    if n > (16 << 20):
        raise ValueError("frame too large")
    mask = b""
    if masked:
        if len(buf) < o + 4:
            return None
        mask, o = buf[o:o + 4], o + 4
    if len(buf) < o + n:
        return None
    payload = buf[o:o + n]
    if masked:
        payload = bytes(b ^ mask[i & 3] for i, b in enumerate(payload))
    return op, payload, o + n


class WebSocketHandler:
    """Text-frame server: every received message is passed to ``on_message(text, send)``; ``send(str)`` writes a frame
    back (call it repeatedly to stream tokens)."""

    def __init__(self, port=8081, on_message: Optional[Callable] = None, host="127.0.0.1"):
        self.port, self.host, self.on_message = port, host, on_message or (lambda text, send: send(text))
        self.sock: Optional[socket.socket] = None
        self._stop = False
        self.clients = 0
        self._socks: List[socket.socket] = []
        self._socks_lock = threading.Lock()

    def is_running(self) -> bool:
        return self.sock is not None and not self._stop

    def broadcast(self, text: str) -> int:
        """Send one text frame to every connected client; returns how many received it (a client whose socket fails is
        dropped)."""
        frame = ws_encode_frame(text.encode())
        with self._socks_lock:
            socks = list(self._socks)
        n = 0
        for c in socks:
            try:
                c.sendall(frame)
                n += 1
            except OSError:
                with self._socks_lock:
                    if c in self._socks:
                        self._socks.remove(c)
        return n

    def start(self):
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.sock.bind((self.host, self.port))
        self.sock.listen(16)
        self.sock.settimeout(0.2)
        self.port = self.sock.getsockname()[1]
        threading.Thread(target=self._accept, daemon=True).start()
        return self.port

    def stop(self):
        self._stop = True
        if self.sock:
            self.sock.close()

    def _accept(self):
        while not self._stop:
            try:
                c, _ = self.sock.accept()
            except (socket.timeout, OSError):
                continue
            threading.Thread(target=self._serve, args=(c,), daemon=True).start()

    def _serve(self, c):
        c.settimeout(30)
        try:
            req = b""
            while b"\r\n\r\n" not in req:
                part = c.recv(4096)
                if not part or len(req) > 65536:
                    return
                req += part
            head, _, rest = req.partition(b"\r\n\r\n")
            hdrs = {}
            for line in head.decode("latin1").split("\r\n")[1:]:
                k, _, v = line.partition(":")
                hdrs[k.strip().lower()] = v.strip()
            key = hdrs.get("sec-websocket-key")
            if hdrs.get("upgrade", "").lower() != "websocket" or not key:
                c.sendall(b"HTTP/1.1 400 Bad Request\r\nContent-Length: 0\r\n\r\n")
                return
            c.sendall(("HTTP/1.1 101 Switching Protocols\r\nUpgrade: websocket\r\nConnection: Upgrade\r\n"
                       f"Sec-WebSocket-Accept: {websocket_accept_key(key)}\r\n\r\n").encode())
            self.clients += 1
            with self._socks_lock:
                self._socks.append(c)
            send = lambda text: c.sendall(ws_encode_frame(text.encode()))
            buf = rest
            while not self._stop:
                fr = ws_decode_frame(buf)
                if fr is None:
                    part = c.recv(65536)
                    if not part:
                        return
                    buf += part
                    continue
                op, payload, used = fr
                buf = buf[used:]
                if op == 8:
                    c.sendall(ws_encode_frame(b"", 8))
                    return
                if op == 9:
                    c.sendall(ws_encode_frame(payload, 10))
                elif op == 1:
                    self.on_message(payload.decode("utf-8", "replace"), send)
        except (OSError, ValueError):
            return
        finally:
            with self._socks_lock:
                if c in self._socks:
                    self._socks.remove(c)
            c.close()


# ================================================================================================ plugins / zoo
class PluginManager:
    """Plugins are Python files (a module with ``plugin_init(ctx)``) or shared libraries (``int plugin_init(void)``,
    optional ``const char* plugin_name(void)``).  ``reload_changed`` re-imports plugins whose file changed."""

    def __init__(self):
        self.plugins: Dict[str, dict] = {}

    def load(self, path: str, ctx=None) -> str:
        name = os.path.splitext(os.path.basename(path))[0]
        if path.endswith(".py"):
            spec = importlib.util.spec_from_file_location(f"tfb_plugin_{name}_{int(time.time() * 1e6)}", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            res = mod.plugin_init(ctx) if hasattr(mod, "plugin_init") else None
            self.plugins[name] = {"path": path, "mtime": os.path.getmtime(path), "module": mod, "result": res, "ctx": ctx, "kind": "python"}
        else:
            lib = ctypes.CDLL(path)
            res = lib.plugin_init() if hasattr(lib, "plugin_init") else None
            if hasattr(lib, "plugin_name"):
                lib.plugin_name.restype = ctypes.c_char_p
                name = lib.plugin_name().decode()
            self.plugins[name] = {"path": path, "mtime": os.path.getmtime(path), "module": lib, "result": res, "ctx": ctx, "kind": "native"}
        return name

    def unload(self, name):
        p = self.plugins.pop(name, None)
        if p and p["kind"] == "python" and hasattr(p["module"], "plugin_shutdown"):
            p["module"].plugin_shutdown()

    def reload_changed(self) -> List[str]:
        out = []
        for name, p in list(self.plugins.items()):
            if p["kind"] == "python" and os.path.getmtime(p["path"]) != p["mtime"]:
                self.unload(name)
                self.load(p["path"], p["ctx"])
                out.append(name)
        return out

    def call(self, name, fn, *args):
        return getattr(self.plugins[name]["module"], fn)(*args)

    # ---- in-process plugins and the generation hooks (reference: Plugin / PluginManager, include/quant/production.h)
    def register_plugin(self, plugin):
        """An object with ``name()`` (or ``name``) and any of on_generate_start / on_token_generated / on_generate_end."""
        if not hasattr(self, "direct"):
            self.direct = []
        self.direct.append(plugin)

    def direct_plugin_count(self) -> int:
        return len(getattr(self, "direct", []))

    def unload_all(self):
        for name in list(self.plugins):
            self.unload(name)
        self.direct = []

    def hot_reload(self, path: str) -> bool:
        """Load ``path`` again in place of the plugin that came from it (or load it for the first time)."""
        for name, p in list(self.plugins.items()):
            if os.path.abspath(p["path"]) == os.path.abspath(path):
                ctx = p["ctx"]
                self.unload(name)
                try:
                    self.load(path, ctx)
                    return True
                except Exception:
                    return False
        try:
            self.load(path)
            return True
        except Exception:
            return False

    def _fire(self, hook: str, arg):
        targets = list(getattr(self, "direct", [])) + [p["module"] for p in self.plugins.values() if p["kind"] == "python"]
        for t in targets:
            fn = getattr(t, hook, None)
            if callable(fn):
                try:
                    fn(arg)
                except Exception:                          # a faulty plugin must not break generation
                    pass

    def on_generate_start(self, prompt: str): self._fire("on_generate_start", prompt)
    def on_token_generated(self, token: int): self._fire("on_token_generated", token)
    def on_generate_end(self, output: str): self._fire("on_generate_end", output)

    def names(self):
        return sorted(self.plugins)


class ModelZoo:
    """name -> checkpoint path registry; models load on first use and can be evicted."""

    def __init__(self, device="cpu", dtype=None):
        self.paths: Dict[str, str] = {}
        self.loaded: Dict[str, object] = {}
        self.device, self.dtype = device, dtype

    def register(self, name, path):
        self.paths[name] = path

    def list(self):
        return sorted(self.paths)

    def get(self, name):
        if name not in self.loaded:
            import torch
            from ..quant import codec
            self.loaded[name] = codec.load_model(self.paths[name], device=self.device, dtype=self.dtype or torch.float32)
        return self.loaded[name]

    def unload(self, name):
        self.loaded.pop(name, None)

    def list_models(self):
        """[{name, path, params, format}] of the registered checkpoints (parameter count and block format read from the
        file's tables, without decoding the weights)."""
        from ..quant import codec
        out = []
        for name in self.list():
            info = {"name": name, "path": self.paths[name], "params": 0, "format": ""}
            try:
                with codec.QuantReader(self.paths[name]) as r:
                    info["params"] = sum(r.block_sizes(b)[0] for b in range(r.num_blocks()))
                    names = r.tensor_names()
                    big = max(names, key=lambda n: r.tensor_blocks(n)[1]) if names else None
                    info["format"] = codec.format_name(r.tensor_format(big)) if big else ""
            except Exception:
                pass
            out.append(info)
        return out

    load = get

    def scan(self, directory):
        for f in sorted(os.listdir(directory)):
            if f.endswith(".quant"):
                self.register(os.path.splitext(f)[0], os.path.join(directory, f))
        return self.list()


class RateLimiter:
    """Token bucket per client key: ``rate`` tokens per second, bursts up to ``burst``.  ``allow`` is what the HTTP front
    end calls before admitting a request (HTTP 429 on refusal); idle buckets are dropped after ``idle_s``.
    Reference counterpart: RateLimiter (src/server/http_server.cpp:116-152); the C++ server has the same policy built in."""

    def __init__(self, rate: float, burst: float, idle_s: float = 300.0, clock=None):
        import threading
        import time as _t
        self.rate, self.burst, self.idle_s = float(rate), float(burst), idle_s
        self._clock = clock or _t.monotonic
        self._b = {}
        self._lock = threading.Lock()

    def allow(self, key: str, cost: float = 1.0) -> bool:
        now = self._clock()
        with self._lock:
            tokens, last = self._b.get(key, (self.burst, now))
            tokens = min(self.burst, tokens + (now - last) * self.rate)
            ok = tokens >= cost
            self._b[key] = (tokens - cost if ok else tokens, now)
            if len(self._b) > 4096:
                self._b = {k: v for k, v in self._b.items() if now - v[1] < self.idle_s}
            return ok

    def retry_after(self, key: str, cost: float = 1.0) -> float:
        with self._lock:
            tokens, last = self._b.get(key, (self.burst, self._clock()))
        return max(0.0, (cost - tokens) / self.rate) if self.rate > 0 else float("inf")

    def set_limits(self, max_requests_per_sec: float, burst: float):
        """New rate and burst for every client; buckets holding more than the new burst are cut down to it."""
        with self._lock:
            self.rate, self.burst = float(max_requests_per_sec), float(burst)
            self._b = {k: (min(t, self.burst), last) for k, (t, last) in self._b.items()}

    def max_requests_per_sec(self) -> float: return self.rate
    def burst_size(self) -> float: return self.burst
