"""GGUF / safetensors / raw importers: files are synthesised byte by byte here and must come back as the
values they encode; a converted checkpoint loads as a model."""
import json
import struct

import numpy as np
import pytest
import torch

from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.quant import codec, importers


def _gguf_str(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _write_gguf(path, tensors, kv=()):
    """tensors: [(name, shape(outer first), ggml type, payload bytes)]"""
    out = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv))
    for k, t, v in kv:
        out += _gguf_str(k) + struct.pack("<I", t)
        out += _gguf_str(v) if t == 8 else struct.pack({4: "<I", 6: "<f"}[t], v)
    off, offs = 0, []
    for name, shape, typ, payload in tensors:
        out += _gguf_str(name) + struct.pack("<I", len(shape))
        for d in reversed(shape):
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", typ, off)
        offs.append(off)
        off += (len(payload) + 31) // 32 * 32
    out += b"\0" * ((-len(out)) % 32)
    for (_, _, _, payload) in tensors:
        out += payload + b"\0" * ((-len(payload)) % 32)
    path.write_bytes(out)


def test_gguf_block_types(tmp_path):
    rng = np.random.default_rng(0)
    f32 = rng.standard_normal(40).astype(np.float32)
    f16 = rng.standard_normal(64).astype(np.float16)
    # Q8_0: 2 blocks
    d8 = np.array([0.5, 0.25], dtype=np.float16)
    q8 = rng.integers(-127, 128, (2, 32)).astype(np.int8)
    p8 = b"".join(d8[i].tobytes() + q8[i].tobytes() for i in range(2))
    # Q4_0: element j in low nibble of byte j, element j+16 in the high nibble
    d4 = np.float16(0.125)
    q4 = rng.integers(0, 16, 32).astype(np.uint8)
    p4 = d4.tobytes() + bytes(int(q4[j]) | (int(q4[j + 16]) << 4) for j in range(16))
    # Q4_1
    m4 = np.float16(-1.0)
    p41 = d4.tobytes() + m4.tobytes() + bytes(int(q4[j]) | (int(q4[j + 16]) << 4) for j in range(16))
    # Q5_0
    q5 = rng.integers(0, 32, 32).astype(np.uint8)
    qh = sum(((int(q5[j]) >> 4) & 1) << j for j in range(32))
    p5 = d4.tobytes() + struct.pack("<I", qh) + bytes((int(q5[j]) & 15) | ((int(q5[j + 16]) & 15) << 4) for j in range(16))
    p51 = d4.tobytes() + m4.tobytes() + struct.pack("<I", qh) + bytes((int(q5[j]) & 15) | ((int(q5[j + 16]) & 15) << 4) for j in range(16))
    bf = torch.randn(8).to(torch.bfloat16)
    _write_gguf(tmp_path / "m.gguf", [
        ("a", (5, 8), 0, f32.tobytes()), ("b", (64,), 1, f16.tobytes()), ("c", (2, 32), 8, p8), ("d", (32,), 2, p4),
        ("e", (32,), 3, p41), ("f", (32,), 6, p5), ("g", (32,), 7, p51), ("h", (8,), 30, bf.view(torch.int16).numpy().tobytes())],
        kv=[("general.architecture", 8, "llama"), ("llama.block_count", 4, 2), ("llama.rope.freq_base", 6, 500000.0)])
    ck = importers.ForeignCheckpoint(tmp_path / "m.gguf")
    assert ck.kind == "gguf" and ck.shape("a") == (5, 8) and ck.dtype("c") == "Q8_0"
    assert ck.metadata()["llama.block_count"] == "2" and float(ck.metadata()["llama.rope.freq_base"]) == 500000.0
    np.testing.assert_array_equal(ck.read("a").numpy().reshape(-1), f32)
    np.testing.assert_array_equal(ck.read("b").numpy(), f16.astype(np.float32))
    np.testing.assert_array_equal(ck.read("c").numpy(), q8.astype(np.float32) * d8.astype(np.float32)[:, None])
    np.testing.assert_array_equal(ck.read("d").numpy(), (q4.astype(np.float32) - 8) * 0.125)
    np.testing.assert_array_equal(ck.read("e").numpy(), q4.astype(np.float32) * 0.125 - 1.0)
    np.testing.assert_array_equal(ck.read("f").numpy(), (q5.astype(np.float32) - 16) * 0.125)
    np.testing.assert_array_equal(ck.read("g").numpy(), q5.astype(np.float32) * 0.125 - 1.0)
    np.testing.assert_array_equal(ck.read("h").numpy(), bf.float().numpy())


def test_gguf_rejects_corrupt(tmp_path):
    (tmp_path / "x.gguf").write_bytes(b"GGUF" + struct.pack("<IQQ", 3, 1 << 40, 0))
    with pytest.raises(ValueError):
        importers.ForeignCheckpoint(tmp_path / "x.gguf")
    (tmp_path / "y.gguf").write_bytes(b"GGUF" + struct.pack("<IQQ", 9, 0, 0))
    with pytest.raises(ValueError, match="version"):
        importers.ForeignCheckpoint(tmp_path / "y.gguf")
    _write_gguf(tmp_path / "z.gguf", [("a", (64,), 0, b"\0" * 16)])     # payload shorter than the shape says
    data = (tmp_path / "z.gguf").read_bytes()
    (tmp_path / "z.gguf").write_bytes(data[:-16])
    with pytest.raises(ValueError, match="truncated"):
        importers.ForeignCheckpoint(tmp_path / "z.gguf").read("a")


def _write_st(path, tensors, meta=None):
    hdr, blob = {}, b""
    for name, (dtype, shape, payload) in tensors.items():
        hdr[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [len(blob), len(blob) + len(payload)]}
        blob += payload
    if meta:
        hdr["__metadata__"] = meta
    h = json.dumps(hdr).encode()
    path.write_bytes(struct.pack("<Q", len(h)) + h + blob)


def test_safetensors_dtypes_and_block_fp8(tmp_path):
    torch.manual_seed(0)
    f = torch.randn(6, 4)
    w8 = (torch.randn(256, 256) * 3).to(torch.float8_e4m3fn)
    sc2d = torch.rand(2, 2) + 0.5
    w8b = torch.randn(300).to(torch.float8_e4m3fn)
    sc1d = torch.rand(3) + 0.5
    e5 = torch.randn(16).to(torch.float8_e5m2)
    _write_st(tmp_path / "m.safetensors", {
        "f32": ("F32", (6, 4), f.numpy().tobytes()),
        "bf16": ("BF16", (6, 4), f.to(torch.bfloat16).view(torch.int16).numpy().tobytes()),
        "f16": ("F16", (6, 4), f.half().numpy().tobytes()),
        "i64": ("I64", (3,), np.array([1, -2, 3], dtype=np.int64).tobytes()),
        "e5": ("F8_E5M2", (16,), e5.view(torch.uint8).numpy().tobytes()),
        "w.weight": ("F8_E4M3", (256, 256), w8.view(torch.uint8).numpy().tobytes()),
        "w.weight_scale_inv": ("F32", (2, 2), sc2d.numpy().tobytes()),
        "v.weight": ("F8_E4M3", (300,), w8b.view(torch.uint8).numpy().tobytes()),
        "v.weight_scale": ("F32", (3,), sc1d.numpy().tobytes())}, meta={"format": "pt"})
    ck = importers.ForeignCheckpoint(tmp_path / "m.safetensors")
    assert ck.kind == "safetensors" and ck.metadata() == {"format": "pt"}
    assert torch.equal(ck.read("f32"), f) and torch.equal(ck.read("bf16"), f.to(torch.bfloat16).float())
    assert torch.equal(ck.read("f16"), f.half().float()) and ck.read("i64").tolist() == [1, -2, 3]
    assert torch.equal(ck.read("e5"), e5.float())
    want = w8.float() * sc2d.repeat_interleave(128, 0).repeat_interleave(128, 1)
    assert torch.equal(ck.read("w.weight"), want)
    assert torch.equal(ck.read("v.weight"), w8b.float() * sc1d.repeat_interleave(128)[:300])
    # header whose offsets disagree with the shape is refused
    _write_st(tmp_path / "bad.safetensors", {"a": ("F32", (4,), b"\0" * 8)})
    with pytest.raises(ValueError, match="shape"):
        importers.ForeignCheckpoint(tmp_path / "bad.safetensors")


def test_convert_hf_names_to_model(tmp_path):
    cfg = TransformerConfig(vocab_size=96, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=128, max_seq_len=64)
    m = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=3)
    inv = {"tok_embeddings.weight": "model.embed_tokens.weight", "norm.weight": "model.norm.weight", "lm_head.weight": "lm_head.weight"}
    tensors = {}
    for name, t in m.named_tensors():
        hf = inv.get(name) or ("model." + name.replace("attention_norm", "input_layernorm").replace("ffn_norm", "post_attention_layernorm")
                               .replace(".attention.", ".self_attn.").replace(".ffn.", ".mlp."))
        tensors[hf] = ("BF16", tuple(t.shape), t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes())
    d = tmp_path / "hf"
    d.mkdir()
    _write_st(d / "model-00001-of-00001.safetensors", tensors)
    (d / "config.json").write_text(json.dumps({"num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 64,
                                                "rope_theta": 10000.0, "rms_norm_eps": 1e-5}))
    rep = importers.convert(str(d), str(tmp_path / "m.quant"))
    assert rep["tensors"] == len(tensors)
    m2 = codec.load_model(tmp_path / "m.quant")
    ids = torch.randint(0, 96, (1, 16))
    with torch.no_grad():
        a, b = m.forward(ids), m2.forward(ids)
    assert (a - b).abs().max() < 0.05
    # budgeted conversion + PTQ + delta
    rep2 = importers.convert(str(d), str(tmp_path / "m5.quant"), target_bpw=5.0)
    assert rep2["bytes"] < rep["bytes"] * 0.35
    hist = importers.ptq_requantize(tmp_path / "m.quant", tmp_path / "m3.quant", 3.0)
    assert hist and (tmp_path / "m3.quant").stat().st_size < (tmp_path / "m5.quant").stat().st_size
    m3 = codec.load_model(tmp_path / "m.quant")
    with torch.no_grad():
        m3.layers[0].o.data.add_(0.01)
    codec.save_model(m3, tmp_path / "tuned.quant")
    assert importers.make_delta(tmp_path / "m.quant", tmp_path / "tuned.quant", tmp_path / "delta.quant", fmt="q16") == 1
    m4 = importers.apply_delta(codec.load_model(tmp_path / "m.quant"), tmp_path / "delta.quant")
    assert (m4.layers[0].o.data - m3.layers[0].o.data).abs().max() < 1e-3


def test_raw_fp32(tmp_path):
    a = np.arange(2048, dtype=np.float32)
    (tmp_path / "w.bin").write_bytes(a.tobytes())
    rep = importers.convert(str(tmp_path / "w.bin"), str(tmp_path / "w.quant"), kind="rawfp32")
    assert rep["weights"] == 2048
    assert torch.equal(codec.QuantReader(tmp_path / "w.quant").read_tensor("weights"), torch.from_numpy(a))
    (tmp_path / "odd.bin").write_bytes(b"123")
    with pytest.raises(ValueError):
        importers.convert(str(tmp_path / "odd.bin"), str(tmp_path / "o.quant"), kind="rawfp32")
