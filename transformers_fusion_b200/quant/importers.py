"""Foreign checkpoints -> ``.quant``: GGUF, safetensors (single file or a sharded model directory, FP8
weights with block scales included) and headerless raw fp32; post-training requantisation to a bit
budget; delta adapters (difference of two checkpoints as a small ``.quant``).

The file parsing and dequantisation are native (csrc/codec/tfb_import.cpp); this module maps tensor
names onto the framework's, infers the model configuration and drives the writer.

Reference counterparts: tools/convert.cpp (raw fp32 :384-444, GGUF :445-553), adapters
safetensors_bridge.h:28-45, tools quant_import / quant_ptq / quant_adapt (src/adapters)."""
from __future__ import annotations

import ctypes as C
import json
import os
import re
from typing import Dict, Iterable, Optional

import numpy as np
import torch

from . import codec
from .planner import FormatPlanner

_BOUND = False


def _lib():
    global _BOUND
    L = codec.lib()
    if not _BOUND:
        L.tfb_import_open.restype = C.c_void_p
        L.tfb_import_open.argtypes = [C.c_char_p, C.c_char_p]
        L.tfb_import_close.argtypes = [C.c_void_p]
        L.tfb_import_error.restype = C.c_char_p
        for n in ("tfb_import_kind", "tfb_import_name", "tfb_import_dtype", "tfb_import_meta_key"):
            getattr(L, n).restype = C.c_char_p
        L.tfb_import_kind.argtypes = [C.c_void_p]
        L.tfb_import_name.argtypes = L.tfb_import_dtype.argtypes = L.tfb_import_meta_key.argtypes = [C.c_void_p, C.c_int]
        L.tfb_import_num_tensors.argtypes = L.tfb_import_num_meta.argtypes = [C.c_void_p]
        L.tfb_import_ndim.argtypes = [C.c_void_p, C.c_int]
        L.tfb_import_dim.restype = L.tfb_import_numel.restype = C.c_longlong
        L.tfb_import_dim.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.tfb_import_numel.argtypes = [C.c_void_p, C.c_int]
        L.tfb_import_find.argtypes = [C.c_void_p, C.c_char_p]
        L.tfb_import_read.restype = L.tfb_import_read_block_fp8.restype = C.c_longlong
        L.tfb_import_read.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_longlong]
        L.tfb_import_read_block_fp8.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong]
        L.tfb_import_meta.restype = C.c_char_p
        L.tfb_import_meta.argtypes = [C.c_void_p, C.c_char_p]
        _BOUND = True
    return L


class ForeignCheckpoint:
    """Read-only view of one GGUF / safetensors / raw-fp32 file."""

    def __init__(self, path, kind="auto"):
        L = _lib()
        self._h = L.tfb_import_open(str(path).encode(), kind.encode())
        if not self._h:
            raise ValueError(L.tfb_import_error().decode())
        self.path = str(path)
        self.kind = L.tfb_import_kind(self._h).decode()
        self.names = [L.tfb_import_name(self._h, i).decode() for i in range(L.tfb_import_num_tensors(self._h))]

    def close(self):
        if getattr(self, "_h", None):
            _lib().tfb_import_close(self._h)
            self._h = None

    __del__ = close

    def __contains__(self, name):
        return _lib().tfb_import_find(self._h, name.encode()) >= 0

    def shape(self, name):
        L, i = _lib(), self._index(name)
        return tuple(L.tfb_import_dim(self._h, i, d) for d in range(L.tfb_import_ndim(self._h, i)))

    def dtype(self, name):
        return _lib().tfb_import_dtype(self._h, self._index(name)).decode()

    def metadata(self) -> Dict[str, str]:
        L = _lib()
        out = {}
        for i in range(L.tfb_import_num_meta(self._h)):
            k = L.tfb_import_meta_key(self._h, i)
            out[k.decode()] = L.tfb_import_meta(self._h, k).decode("utf-8", "replace")
        return out

    def _index(self, name):
        i = _lib().tfb_import_find(self._h, name.encode())
        if i < 0:
            raise KeyError(name)
        return i

    def read(self, name, fp8_block=128) -> torch.Tensor:
        """fp32 tensor; an FP8 weight with a ``<name>_scale_inv`` / ``<name>_scale`` companion is scaled by it."""
        L, i = _lib(), self._index(name)
        n = L.tfb_import_numel(self._h, i)
        out = np.empty(max(1, n), dtype=np.float32)
        scale = next((s for s in (name + "_scale_inv", name + "_scale") if s in self), None)
        if scale is not None and self.dtype(name).startswith("F8"):
            got = L.tfb_import_read_block_fp8(self._h, i, self._index(scale), fp8_block, out.ctypes.data, n)
        else:
            got = L.tfb_import_read(self._h, i, out.ctypes.data, n)
        if got != n:
            raise ValueError(L.tfb_import_error().decode())
        return torch.from_numpy(out[:n]).view(self.shape(name))


# ---------------------------------------------------------------------------------------------- name mapping
_HF_RULES = [
    (r"^model\.embed_tokens\.weight$", "tok_embeddings.weight"),
    (r"^model\.norm\.weight$", "norm.weight"),
    (r"^lm_head\.weight$", "lm_head.weight"),
    (r"^model\.layers\.(\d+)\.input_layernorm\.weight$", r"layers.\1.attention_norm.weight"),
    (r"^model\.layers\.(\d+)\.post_attention_layernorm\.weight$", r"layers.\1.ffn_norm.weight"),
    (r"^model\.layers\.(\d+)\.self_attn\.([qkvo])_proj\.(weight|bias)$", r"layers.\1.attention.\2_proj.\3"),
    (r"^model\.layers\.(\d+)\.mlp\.(gate|up|down)_proj\.weight$", r"layers.\1.ffn.\2_proj.weight"),
    (r"^model\.layers\.(\d+)\.mlp\.gate\.weight$", r"layers.\1.moe.router.weight"),
    (r"^model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$", r"layers.\1.moe.experts.\2.\3_proj.weight"),
    (r"^model\.layers\.(\d+)\.mlp\.shared_experts?\.(gate|up|down)_proj\.weight$", r"layers.\1.moe.shared.\2_proj.weight"),
]
_GGUF_RULES = [
    (r"^token_embd\.weight$", "tok_embeddings.weight"),
    (r"^output_norm\.weight$", "norm.weight"),
    (r"^output\.weight$", "lm_head.weight"),
    (r"^blk\.(\d+)\.attn_norm\.weight$", r"layers.\1.attention_norm.weight"),
    (r"^blk\.(\d+)\.ffn_norm\.weight$", r"layers.\1.ffn_norm.weight"),
    (r"^blk\.(\d+)\.attn_(q|k|v)\.(weight|bias)$", r"layers.\1.attention.\2_proj.\3"),
    (r"^blk\.(\d+)\.attn_output\.(weight|bias)$", r"layers.\1.attention.o_proj.\2"),
    (r"^blk\.(\d+)\.ffn_(gate|up|down)\.weight$", r"layers.\1.ffn.\2_proj.weight"),
]


def map_name(name: str) -> Optional[str]:
    """Framework tensor name for a HuggingFace / GGUF tensor name (None: not part of the decoder)."""
    for pat, rep in _HF_RULES + _GGUF_RULES:
        if re.match(pat, name):
            return re.sub(pat, rep, name)
    if name.startswith(("layers.", "tok_embeddings.", "norm.", "lm_head.", "pos_embeddings.", "mtp_heads.")):
        return name
    return None


def infer_config(tensors: Dict[str, tuple], meta: Dict[str, str] = None, hf_config: dict = None):
    """TransformerConfig from tensor shapes (+ GGUF metadata / HF config.json for heads, rope and eps)."""
    from ..models.config import TransformerConfig
    meta, hf = meta or {}, hf_config or {}
    V, H = tensors["tok_embeddings.weight"]
    L = 1 + max(int(m.group(1)) for m in (re.match(r"layers\.(\d+)\.", n) for n in tensors) if m)
    arch = meta.get("general.architecture", "llama")

    def g(key, hf_key, default):
        if hf_key in hf:
            return hf[hf_key]
        v = meta.get(f"{arch}.{key}")
        return type(default)(float(v)) if v is not None else default
    q_rows = tensors["layers.0.attention.q_proj.weight"][0]
    kv_rows = tensors["layers.0.attention.k_proj.weight"][0]
    heads = int(g("attention.head_count", "num_attention_heads", max(1, q_rows // 128) if q_rows % 128 == 0 else max(1, q_rows // 64)))
    D = hf.get("head_dim", q_rows // heads)
    kv = int(g("attention.head_count_kv", "num_key_value_heads", kv_rows // D))
    F = tensors["layers.0.ffn.up_proj.weight"][0] if "layers.0.ffn.up_proj.weight" in tensors else 4 * H
    gated = "layers.0.ffn.gate_proj.weight" in tensors
    return TransformerConfig(vocab_size=V, hidden_size=H, num_layers=L, num_heads=heads, num_kv_heads=kv, ffn_hidden_size=F,
                             max_seq_len=int(g("context_length", "max_position_embeddings", 2048)),
                             rope_theta=float(g("rope.freq_base", "rope_theta", 10000.0)),
                             norm_eps=float(g("attention.layer_norm_rms_epsilon", "rms_norm_eps", 1e-5)),
                             activation="swiglu" if gated else "gelu", tie_embeddings="lm_head.weight" not in tensors,
                             head_dim=int(D), attention_bias="layers.0.attention.q_proj.bias" in tensors)


def _sources(path) -> Iterable[ForeignCheckpoint]:
    if os.path.isdir(path):
        files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        if not files:
            raise ValueError(f"{path}: no .safetensors files")
        for f in files:
            yield ForeignCheckpoint(os.path.join(path, f), "safetensors")
    else:
        yield ForeignCheckpoint(path)


def convert(input_path, output_path, kind="auto", target_bpw: float = 0.0, fmt: Optional[str] = None, verbose=False):
    """Any supported foreign checkpoint -> ``.quant``.  ``target_bpw`` > 0 plans a per-block format mix
    for every matrix (norms, biases and tensors under 1024 weights stay fp32); ``fmt`` forces one format;
    neither: fp32 pass-through.  Returns {"tensors", "weights", "bytes", "bpw"}."""
    srcs = [ForeignCheckpoint(input_path, kind)] if not os.path.isdir(input_path) else list(_sources(input_path))
    hf_cfg = {}
    cfg_path = os.path.join(input_path if os.path.isdir(input_path) else os.path.dirname(input_path) or ".", "config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            hf_cfg = json.load(f)
    shapes, owner, meta = {}, {}, {}
    for s in srcs:
        meta.update(s.metadata())
        for n in s.names:
            m = map_name(n) if s.kind != "rawfp32" else n
            if m is None or n.endswith(("_scale_inv", "_scale")):
                continue
            shapes[m], owner[m] = s.shape(n), (s, n)
    config = b""
    if "tok_embeddings.weight" in shapes and "layers.0.attention.q_proj.weight" in shapes:
        config = infer_config(shapes, meta, hf_cfg).to_bytes()
    forced = codec.parse_format(fmt) if fmt else -1
    if fmt and forced < 0:
        raise ValueError(f"unknown format '{fmt}'")
    w = codec.QuantWriter(output_path, config)
    total = 0
    for name, (s, n) in owner.items():
        t = s.read(n)
        total += t.numel()
        small = t.numel() < 1024 or (t.dim() < 2 and s.kind != "rawfp32")
        if verbose:
            print(f"  {n} -> {name} {tuple(t.shape)} {s.dtype(n)}")
        if small or (forced < 0 and target_bpw <= 0):
            w.add_tensor(name, t, codec.Q_32)
        elif forced >= 0:
            w.add_tensor(name, t, forced)
        else:
            p = FormatPlanner(target_bpw)
            p.score_importance(t)
            w.add_tensor_mixed(name, t, p.plan_for_model(t.numel()).formats())
    w.close()
    for s in srcs:
        s.close()
    size = os.path.getsize(output_path)
    return {"tensors": len(owner), "weights": total, "bytes": size, "bpw": 8.0 * size / max(1, total)}


# ---------------------------------------------------------------------------------------------- PTQ
def ptq_requantize(input_quant, output_quant, target_bpw: float, importance: Optional[Dict[str, torch.Tensor]] = None,
                   metric="magnitude", keep_fp32=("norm", "bias")):
    """Post-training requantisation of a ``.quant`` file to a bit budget.  ``importance`` optionally maps
    tensor names to calibration activations (magnitude metric) or gradients (``metric='fisher_diag'``) of the
    same shape; blocks that matter most keep the precise tier.  Returns the per-tensor plans' histograms."""
    r = codec.QuantReader(input_quant)
    w = codec.QuantWriter(output_quant, r.config_bytes(), r.version)
    report = {}
    for name in r.tensor_names():
        t = r.read_tensor(name)
        if t.numel() < 1024 or any(k in name for k in keep_fp32):
            w.add_tensor(name, t, codec.Q_32)
            continue
        p = FormatPlanner(target_bpw)
        p.score_importance(t, (importance or {}).get(name), metric=metric if importance and name in importance else "magnitude")
        plan = p.plan_for_model(t.numel())
        w.add_tensor_mixed(name, t, plan.formats())
        report[name] = plan.histogram()
    w.close()
    r.close()
    return report


# ---------------------------------------------------------------------------------------------- delta adapters
def make_delta(base_quant, tuned_quant, output_quant, fmt="q8", min_rel_change=1e-6):
    """Store ``tuned - base`` for every tensor that changed; unchanged tensors are left out."""
    b, t = codec.QuantReader(base_quant), codec.QuantReader(tuned_quant)
    w = codec.QuantWriter(output_quant, t.config_bytes(), t.version, flags=1)
    f = codec.parse_format(fmt)
    kept = 0
    for name in t.tensor_names():
        tv = t.read_tensor(name)
        try:
            d = tv - b.read_tensor(name)
        except KeyError:
            d = tv
        if float(d.abs().max()) <= min_rel_change * max(1e-30, float(tv.abs().max())):
            continue
        w.add_tensor(name, d, f if d.numel() >= 1024 else codec.Q_32)
        kept += 1
    w.close()
    return kept


def apply_delta(model, delta_quant, scale: float = 1.0):
    """Add a delta adapter onto a loaded model in place."""
    with codec.QuantReader(delta_quant) as r:
        names = set(r.tensor_names())
        with torch.no_grad():
            for name, dst in model.named_tensors():
                if name in names:
                    dst.add_((scale * r.read_tensor(name)).view(dst.shape).to(device=dst.device, dtype=dst.dtype))
    return model
