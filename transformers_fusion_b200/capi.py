"""Python side of the C API (csrc/capi/tfb_capi.cpp): ``load(path)`` returns a handle whose ``generate`` the C entry
point calls.  Also usable directly from Python as a minimal "load and generate" facade."""
from __future__ import annotations

import os


class Handle:
    def __init__(self, path: str):
        import torch

        from .cli.common import load_tokenizer, model_dtype, pick_device
        from .inference.engine import EngineConfig, InferenceEngine
        from .quant import codec
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        dev = pick_device(os.environ.get("TFB_DEVICE", "auto"))
        self.model = codec.load_model(path, device=dev, dtype=model_dtype(dev))
        self.tok = load_tokenizer(path)
        self.engine = InferenceEngine(self.model, self.tok, EngineConfig(num_pages=max(64, 4 * self.model.cfg.max_seq_len // 16)))

    def generate(self, prompt: str, max_tokens: int, temperature: float, top_k: int, top_p: float) -> str:
        from .inference.sampler import SamplerConfig
        max_tokens = max(1, min(int(max_tokens), self.model.cfg.max_seq_len - 2))
        return self.engine.generate(prompt, max_tokens, SamplerConfig(float(temperature), int(top_k), float(top_p)))


def load(path: str) -> Handle:
    return Handle(path)
