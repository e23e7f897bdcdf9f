"""quant_serve / quant_server: OpenAI-compatible HTTP server over the native front end and the
continuous-batching engine.  ``--model --port(8080) --batch-size --workers(4) --max-tokens`` (tools/serve.cpp:18-148)
plus ``--model-dir --temperature --top-k --top-p`` (tools/quant_server.cpp:50-80) and ``--kv --auth-token``."""
from __future__ import annotations

import argparse
import signal
import sys
import threading
import time

from .common import add_float, add_int, load_tokenizer, model_dtype, pick_device


class EngineService:
    """Thread-safe bridge between HTTP worker threads and the single engine loop (continuous batching)."""

    def __init__(self, engine, defaults):
        self.engine, self.defaults = engine, defaults
        self.lock = threading.Lock()
        self.cv = threading.Condition(self.lock)
        self.running = True
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        while self.running:
            with self.cv:
                while self.running and (self.engine is None or not self.engine.has_pending()):
                    self.cv.wait(0.05)
                if not self.running:
                    return
                self.engine.step()
                self.cv.notify_all()

    def generate(self, prompt, max_tokens, temperature, top_p, top_k, stream):
        from ..inference.sampler import SamplerConfig
        eng = self.engine                       # a model swap waits for this request: it is pending on `eng` until it ends
        if eng is None:
            raise RuntimeError("no model is loaded")
        tok = eng.tok
        ids = tok.encode(prompt)[-(eng.max_len - 2):] or [tok.bos_id if tok.bos_id >= 0 else 0]
        pieces, acc, sent = [], [], [""]

        def on_tok(t):
            if t == tok.eos_id:
                return
            acc.append(t)
            text = tok.decode(acc)
            if not text.endswith("�"):
                pieces.append(text[len(sent[0]):])
                sent[0] = text
        sc = SamplerConfig(temperature, top_k, top_p)
        with self.cv:
            if self.engine is not eng:          # swapped between the two lines above
                eng = self.engine
                if eng is None:
                    raise RuntimeError("no model is loaded")
            r = eng.add_request(ids, min(max_tokens, self.defaults["max_tokens"]), sc, on_token=on_tok)
            self.cv.notify_all()
        emitted = 0
        while True:
            with self.cv:
                while emitted >= len(pieces) and not r.finished:
                    self.cv.wait(0.05)
                new, done = pieces[emitted:], r.finished
                emitted = len(pieces)
            for p in new:
                if p:
                    yield p
            if done and emitted >= len(pieces):
                break
        self.last_usage = (len(ids), len(r.out))

    def swap_engine(self, engine):
        """Serve from another engine: waits until the current one has nothing in flight, under the loop's lock."""
        with self.cv:
            while self.engine is not None and self.engine.has_pending():
                self.cv.wait(0.05)
            self.engine = engine
            self.cv.notify_all()

    def stop(self):
        self.running = False
        with self.cv:
            self.cv.notify_all()


def main(argv=None):
    ap = argparse.ArgumentParser(prog="quant_serve")
    ap.add_argument("--model", required=True)
    ap.add_argument("--model-dir", default="")
    add_int(ap, "--port", 8080)
    add_int(ap, "--batch-size", 64)
    add_int(ap, "--workers", 4)
    add_int(ap, "--max-tokens", 2048)
    add_float(ap, "--temperature", 0.7)
    add_int(ap, "--top-k", 40)
    add_float(ap, "--top-p", 0.9)
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8", "q4"])
    ap.add_argument("--auth-token", default="")
    ap.add_argument("--weights", default="", choices=["", "int8", "int4", "mxfp8", "fp4", "ternary"])
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    from ..inference.engine import EngineConfig, InferenceEngine
    from ..quant import codec
    from ..server import HTTPServer
    dev = pick_device(a.device)
    def build_engine(path):
        model = codec.load_model(path, device=dev, dtype=model_dtype(dev))
        tok = load_tokenizer(path, a.model_dir)
        return InferenceEngine(model, tok, EngineConfig(max_batch=a.batch_size, kv_mode=a.kv, num_pages=4096, weight_format=a.weights))
    eng = build_engine(a.model)
    svc = EngineService(eng, {"max_tokens": a.max_tokens})
    srv = HTTPServer(a.port)
    srv.set_thread_pool_size(max(a.workers, a.batch_size))
    srv.set_model_name(a.model)
    if a.auth_token:
        srv.set_auth_token(a.auth_token)
    srv.set_generate_callback(lambda p, mt, t, tp, tk, st: svc.generate(p, mt, t, tp, tk, st))

    def embed(text):
        import torch
        e = svc.engine
        if e is None:
            raise RuntimeError("no model is loaded")
        ids = torch.tensor([e.tok.encode(text)[: e.max_len] or [0]], device=dev)
        with torch.no_grad():
            return e.model.hidden_states(ids).float().mean(0).tolist()
    srv.set_embeddings_callback(embed)

    def load(path):                                   # POST /v1/models/load: build first, swap when the old engine is idle
        try:
            svc.swap_engine(build_engine(path))
            return True
        except Exception as e:                        # a bad path or file leaves the current model in service
            print(f"load {path}: {e}", file=sys.stderr, flush=True)
            return False
    srv.set_load_model_callback(load)
    srv.set_unload_model_callback(lambda: svc.swap_engine(None))
    if not srv.start():
        print(f"Error: cannot bind port {a.port}", file=sys.stderr)
        return 1
    print(f"Serving {a.model} on port {srv.port} ({a.workers} workers)", flush=True)
    stop = threading.Event()
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: stop.set())
    while not stop.is_set():
        time.sleep(0.2)
    srv.stop()
    svc.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
