"""HTTP serving front end: Python binding of ``libtfb_serve`` (the native OpenAI-compatible server).

``HTTPServer`` mirrors the reference class (include/quant/http_server.h:60-213): ``start/stop/
is_running``, ``set_thread_pool_size``, ``set_timeout_seconds``, ``set_max_body_size``,
``set_rate_limit(rps, burst)``, ``set_auth_token``, ``set_max_header_bytes``, ``set_max_concurrent``,
``set_model_name``, ``set_generate_callback``, ``set_embeddings_callback`` and the three static
wire helpers ``openai_error_json``, ``sse_data_frame``, ``sse_done_frame``."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB = None
_EMIT = C.CFUNCTYPE(None, C.c_void_p, C.c_char_p)
_GEN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_char_p, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int, _EMIT, C.c_void_p,
                   C.POINTER(C.c_int), C.POINTER(C.c_int))
_EMB = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_char_p, C.POINTER(C.c_float), C.c_int)
_LOAD = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_char_p)
_UNLOAD = C.CFUNCTYPE(None, C.c_void_p)


def _lib():
    global _LIB
    if _LIB is None:
        p = Path(__file__).resolve().parent.parent / "lib" / "libtfb_serve.so"
        if not p.exists():
            from .. import build
            build.build_host_lib("tfb_serve", "serve")
        L = C.CDLL(str(p))
        L.tfb_server_new.restype = C.c_void_p
        L.tfb_server_new.argtypes = [C.c_int]
        for n in ("tfb_server_free", "tfb_server_stop"):
            getattr(L, n).argtypes = [C.c_void_p]
            getattr(L, n).restype = None
        for n in ("tfb_server_start", "tfb_server_is_running", "tfb_server_current_requests", "tfb_server_port",
                  "tfb_server_max_header", "tfb_server_max_concurrent"):
            getattr(L, n).argtypes = [C.c_void_p]
        for n in ("tfb_server_set_workers", "tfb_server_set_timeout", "tfb_server_set_max_header",
                  "tfb_server_set_max_concurrent"):
            getattr(L, n).argtypes = [C.c_void_p, C.c_int]
            getattr(L, n).restype = None
        for n in ("tfb_server_total_requests", "tfb_server_total_errors", "tfb_server_total_tokens"):
            getattr(L, n).argtypes = [C.c_void_p]
            getattr(L, n).restype = C.c_longlong
        L.tfb_server_model_name.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        L.tfb_server_set_max_body.argtypes = [C.c_void_p, C.c_longlong]
        L.tfb_server_set_rate_limit.argtypes = [C.c_void_p, C.c_double, C.c_double]
        L.tfb_server_set_auth_token.argtypes = [C.c_void_p, C.c_char_p]
        L.tfb_server_set_model_name.argtypes = [C.c_void_p, C.c_char_p]
        L.tfb_server_set_generate.argtypes = [C.c_void_p, _GEN, C.c_void_p]
        L.tfb_server_set_embeddings.argtypes = [C.c_void_p, _EMB, C.c_void_p]
        L.tfb_server_set_model_callbacks.argtypes = [C.c_void_p, _LOAD, _UNLOAD, C.c_void_p]
        L.tfb_server_set_model_callbacks.restype = None
        L.tfb_server_latency_pct.restype = C.c_double
        L.tfb_server_latency_pct.argtypes = [C.c_void_p, C.c_double]
        L.tfb_server_ttft_pct.restype = C.c_double
        L.tfb_server_ttft_pct.argtypes = [C.c_void_p, C.c_double]
        L.tfb_openai_error_json.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_int]
        L.tfb_sse_data_frame.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        L.tfb_sse_done_frame.restype = C.c_char_p
        _LIB = L
    return _LIB


class HTTPServer:
    def __init__(self, port: int = 8080):
        self._h = _lib().tfb_server_new(port)
        self._auth = ""
        self._keep = []

    # ---- lifecycle
    def start(self) -> bool:
        return _lib().tfb_server_start(self._h) == 0

    def stop(self):
        if self._h:
            _lib().tfb_server_stop(self._h)

    def is_running(self) -> bool:
        return bool(_lib().tfb_server_is_running(self._h))

    @property
    def port(self) -> int:
        return _lib().tfb_server_port(self._h)

    def current_requests(self) -> int:
        return _lib().tfb_server_current_requests(self._h)

    def total_requests(self) -> int: return _lib().tfb_server_total_requests(self._h)
    def total_errors(self) -> int: return _lib().tfb_server_total_errors(self._h)
    def total_tokens(self) -> int: return _lib().tfb_server_total_tokens(self._h)

    def model_name(self) -> str:
        """The name the server reports, including one set by a ``/v1/models/load`` request."""
        buf = C.create_string_buffer(512)
        _lib().tfb_server_model_name(self._h, buf, 512)
        return buf.value.decode("utf-8", "replace")

    def __del__(self):
        if getattr(self, "_h", None):
            _lib().tfb_server_stop(self._h)
            _lib().tfb_server_free(self._h)
            self._h = None

    # ---- configuration
    def set_thread_pool_size(self, n): _lib().tfb_server_set_workers(self._h, n)
    def set_timeout_seconds(self, s): _lib().tfb_server_set_timeout(self._h, s)
    def set_max_body_size(self, n): _lib().tfb_server_set_max_body(self._h, n)
    def set_rate_limit(self, rps, burst): _lib().tfb_server_set_rate_limit(self._h, float(rps), float(burst))
    def set_max_header_bytes(self, n): _lib().tfb_server_set_max_header(self._h, n)
    def max_header_bytes(self): return _lib().tfb_server_max_header(self._h)
    def set_max_concurrent(self, n): _lib().tfb_server_set_max_concurrent(self._h, n)
    def max_concurrent(self): return _lib().tfb_server_max_concurrent(self._h)
    def set_model_name(self, n): _lib().tfb_server_set_model_name(self._h, n.encode())

    def set_auth_token(self, t):
        self._auth = t
        _lib().tfb_server_set_auth_token(self._h, t.encode())

    def auth_token(self):
        return self._auth

    def latency_ms(self, pct=0.5): return _lib().tfb_server_latency_pct(self._h, pct)
    def ttft_ms(self, pct=0.5): return _lib().tfb_server_ttft_pct(self._h, pct)

    # ---- callbacks
    def set_generate_callback(self, fn):
        """``fn(prompt, max_tokens, temperature, top_p, top_k, stream)`` returns the completion as a string,
        an iterable of text pieces (streamed as they are produced), or a tuple (pieces, prompt_tokens,
        completion_tokens)."""
        def tramp(_u, prompt, max_tokens, temperature, top_p, top_k, stream, emit, ectx, pt, ct):
            try:
                out = fn(prompt.decode("utf-8", "replace"), max_tokens, temperature, top_p, top_k, bool(stream))
                usage = None
                if isinstance(out, tuple):
                    out, usage = out[0], out[1:]
                n = 0
                for piece in ([out] if isinstance(out, str) else out):
                    emit(ectx, piece.encode("utf-8"))
                    n += 1
                if usage:
                    pt[0], ct[0] = int(usage[0]), int(usage[1])
                else:
                    ct[0] = n
                return 0
            except Exception:  # reported to the client as a 500, never propagated into the C++ worker
                return 1
        cb = _GEN(tramp)
        self._keep.append(cb)
        _lib().tfb_server_set_generate(self._h, cb, None)

    def set_load_model_callback(self, fn):
        """``fn(path) -> bool``: called by ``POST /v1/models/load {"path": ..., "name": ...}``; a true result makes the
        model at ``path`` the served one (reference: HTTPServer::set_load_model_callback, include/quant/http_server.h:125)."""
        self._load_fn = fn
        self._install_model_callbacks()

    def set_unload_model_callback(self, fn):
        """``fn()``: called by ``POST /v1/models/unload``; until the next load, generation answers 503."""
        self._unload_fn = fn
        self._install_model_callbacks()

    def _install_model_callbacks(self):
        load_fn, unload_fn = getattr(self, "_load_fn", None), getattr(self, "_unload_fn", None)

        def load_tramp(_u, path):
            try:
                return 1 if load_fn(path.decode("utf-8", "replace")) else 0
            except Exception:
                return 0

        def unload_tramp(_u):
            try:
                unload_fn()
            except Exception:
                pass
        lcb = _LOAD(load_tramp) if load_fn else C.cast(None, _LOAD)
        ucb = _UNLOAD(unload_tramp) if unload_fn else C.cast(None, _UNLOAD)
        self._keep += [lcb, ucb]
        _lib().tfb_server_set_model_callbacks(self._h, lcb, ucb, None)

    def set_embeddings_callback(self, fn):
        def tramp(_u, text, out, cap):
            try:
                v = fn(text.decode("utf-8", "replace"))
                n = min(len(v), cap)
                for i in range(n):
                    out[i] = float(v[i])
                return n
            except Exception:
                return -1
        cb = _EMB(tramp)
        self._keep.append(cb)
        _lib().tfb_server_set_embeddings(self._h, cb, None)

    # ---- wire helpers (exact bytes)
    @staticmethod
    def openai_error_json(message, type_="", code=""):
        buf = C.create_string_buffer(4096 + 2 * len(message))
        _lib().tfb_openai_error_json(message.encode(), type_.encode(), code.encode(), buf, len(buf))
        return buf.value.decode()

    @staticmethod
    def sse_data_frame(json_text):
        buf = C.create_string_buffer(len(json_text.encode()) + 16)
        _lib().tfb_sse_data_frame(json_text.encode(), buf, len(buf))
        return buf.value.decode()

    @staticmethod
    def sse_done_frame():
        return _lib().tfb_sse_done_frame().decode()
