"""Text-in / text-out inference facade over the paged engine: load a checkpoint with its vocabulary, generate with
statistics, stream with punctuation-aligned flushing, batch prompts.

Reference counterparts: engine::InferenceEngine (engines/inference/inference.h:13-75, inference.cpp:47-200), StreamBuffer
(engines/inference/stream.cpp:10-33)."""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Tuple

from ..inference import engine as _E
from ..inference.sampler import SamplerConfig

_FLUSH = set(" \n\t.,!?;:)}]\"'\r")


class StreamBuffer:
    """Collects token text and releases it at word / punctuation boundaries so that a consumer never sees half a word."""

    def __init__(self):
        self.buffer = ""

    def append(self, text: str): self.buffer += text
    def should_flush(self) -> bool: return bool(self.buffer) and self.buffer[-1] in _FLUSH

    def flush(self, sink: Callable[[str], None]):
        if self.buffer:
            sink(self.buffer)
            self.buffer = ""


@dataclass
class EngineConfig:
    max_seq_len: int = 2048
    num_threads: int = 1               # accepted for compatibility; the device engine has no host thread pool
    use_fp16: bool = False             # accepted for compatibility; compute is bf16
    use_kv_cache: bool = True          # the paged cache is always on; False only disables prefix sharing
    kv_mode: str = "bf16"
    max_tokens: int = 512
    sampler: SamplerConfig = field(default_factory=lambda: SamplerConfig(temperature=0.7, top_k=40, top_p=0.9))


@dataclass
class InferenceStats:
    tokens_generated: int = 0
    duration_sec: float = 0.0
    tokens_per_sec: float = 0.0
    peak_memory_bytes: int = 0
    kv_cache_utilization: float = 0.0


class InferenceEngine:
    def __init__(self):
        self.model = self.tokenizer = self._eng = None
        self._cfg = EngineConfig()
        self._stats = InferenceStats()

    # ---------------------------------------------------------------- set-up
    def load(self, quant_path: str, device: Optional[str] = None) -> Tuple[bool, str]:
        """Loads ``model.quant`` and the vocabulary beside it (``model.vocab`` or ``model.quant.vocab``)."""
        import torch
        from ..cli.common import load_tokenizer
        from ..quant.codec import load_model
        if not os.path.exists(quant_path):
            return False, f"no such file: {quant_path}"
        try:
            dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
            model = load_model(quant_path, device=dev)
            tok = load_tokenizer(quant_path, os.path.dirname(quant_path) or ".")
        except (OSError, ValueError, RuntimeError) as e:
            return False, str(e)
        self.init(model, tok, self._cfg)
        return True, ""

    def init(self, model, tokenizer, cfg: Optional[EngineConfig] = None):
        self.model, self.tokenizer = model, tokenizer
        self._cfg = cfg or self._cfg
        c = self._cfg
        self._eng = _E.InferenceEngine(model, tokenizer, _E.EngineConfig(max_seq_len=c.max_seq_len, kv_mode=c.kv_mode,
                                                                         enable_prefix_cache=c.use_kv_cache))
        return self

    def config(self) -> EngineConfig: return self._cfg
    def last_stats(self) -> InferenceStats: return self._stats

    # ---------------------------------------------------------------- generation
    def _update(self, n_tokens: int, dt: float):
        import torch
        s = self._stats
        s.tokens_generated, s.duration_sec = n_tokens, dt
        s.tokens_per_sec = n_tokens / dt if dt > 0 else 0.0
        if torch.cuda.is_available():
            s.peak_memory_bytes = int(torch.cuda.max_memory_allocated())
        alloc = self._eng.cache.allocator
        s.kv_cache_utilization = 1.0 - alloc.num_free / max(1, alloc.num_pages)

    def generate(self, prompt: str) -> str:
        return self.generate_with_stats(prompt)[0]

    def generate_with_stats(self, prompt: str) -> Tuple[str, InferenceStats]:
        if self._eng is None:
            return "", self._stats
        t0 = time.perf_counter()
        before = self._eng.stats.generated_tokens
        text = self._eng.generate(prompt, self._cfg.max_tokens, self._cfg.sampler)
        self._update(self._eng.stats.generated_tokens - before, time.perf_counter() - t0)
        return text, self._stats

    def generate_stream(self, prompt: str, on_token: Callable[[str], None]):
        if self._eng is None:
            return
        sb = StreamBuffer()
        t0 = time.perf_counter()
        before = self._eng.stats.generated_tokens

        def buffered(piece: str):
            sb.append(piece)
            if sb.should_flush():
                sb.flush(on_token)
        self._eng.generate_stream(prompt, buffered, self._cfg.max_tokens, self._cfg.sampler)
        sb.flush(on_token)
        self._update(self._eng.stats.generated_tokens - before, time.perf_counter() - t0)

    def generate_batch(self, prompts: List[str]) -> List[str]:
        if self._eng is None:
            return ["" for _ in prompts]
        t0 = time.perf_counter()
        before = self._eng.stats.generated_tokens
        outs = self._eng.generate_batch([self.tokenizer.encode(p) for p in prompts], self._cfg.max_tokens, self._cfg.sampler)
        self._update(self._eng.stats.generated_tokens - before, time.perf_counter() - t0)
        eos = self.tokenizer.eos_id
        return [self.tokenizer.decode([t for t in o if t != eos]) for o in outs]

    def reset_context(self):
        if self._eng is not None:
            self._eng.reset_context()
