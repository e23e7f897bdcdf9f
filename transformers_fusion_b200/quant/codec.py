"""Python binding of ``libtfb_codec`` (format registry, block codec, ``.quant`` container, ``.opt``).

``Format`` ids, names and wire bits-per-weight follow the reference enum (include/quant/types.h:22-277).
``save_model`` / ``load_model`` use the reference's tensor names and block sizes (32768-weight Q_32
blocks for full-precision saves, 256-weight blocks for quantised ones: src/model/model.cpp:168-331)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np
import torch

_LIB = None
FORMAT_COUNT = 105
Q_32 = 9


def lib():
    global _LIB
    if _LIB is None:
        p = Path(__file__).resolve().parent.parent / "lib" / "libtfb_codec.so"
        if not p.exists():
            from .. import build
            build.build_host_lib("tfb_codec", "codec")
        L = C.CDLL(str(p))
        L.tfb_format_name.restype = C.c_char_p
        L.tfb_format_name.argtypes = [C.c_int]
        L.tfb_format_parse.argtypes = [C.c_char_p]
        L.tfb_format_bpw.restype = C.c_double
        L.tfb_format_bpw.argtypes = [C.c_int]
        L.tfb_block_claimed_bytes.restype = C.c_size_t
        L.tfb_block_claimed_bytes.argtypes = [C.c_int, C.c_uint32]
        L.tfb_quantize_block.restype = C.c_long
        L.tfb_quantize_block.argtypes = [C.c_int, C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t]
        L.tfb_dequantize_block.restype = None
        L.tfb_dequantize_block.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_uint32, C.c_void_p]
        L.tfb_sha256.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.tfb_reader_open.restype = C.c_void_p
        L.tfb_reader_open.argtypes = [C.c_char_p]
        for n in ("tfb_reader_valid", "tfb_reader_version", "tfb_reader_flags", "tfb_reader_num_tensors",
                  "tfb_reader_num_blocks"):
            getattr(L, n).argtypes = [C.c_void_p]
        L.tfb_reader_close.argtypes = [C.c_void_p]
        L.tfb_reader_config.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32]
        L.tfb_reader_tensor_name.restype = C.c_char_p
        L.tfb_reader_tensor_name.argtypes = [C.c_void_p, C.c_uint32]
        L.tfb_reader_tensor_numel.restype = C.c_longlong
        L.tfb_reader_tensor_numel.argtypes = [C.c_void_p, C.c_char_p]
        L.tfb_reader_tensor_format.argtypes = [C.c_void_p, C.c_char_p]
        L.tfb_reader_read_tensor.restype = C.c_longlong
        L.tfb_reader_read_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_longlong]
        L.tfb_writer_open.restype = C.c_void_p
        L.tfb_writer_open.argtypes = [C.c_char_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32]
        L.tfb_writer_add_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_longlong, C.c_int, C.c_uint32]
        L.tfb_writer_close.argtypes = [C.c_void_p, C.c_int]
        L.tfb_writer_add_tensor_mixed.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_uint32,
                                                  C.c_uint32]
        L.tfb_reader_tensor_range.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_void_p]
        L.tfb_reader_block_info.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p]
        L.tfb_reader_block_payload.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]
        L.tfb_reader_decode_block.restype = C.c_longlong
        L.tfb_reader_decode_block.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_longlong]
        L.tfb_reader_block_offset.restype = C.c_longlong
        L.tfb_reader_block_offset.argtypes = [C.c_void_p, C.c_uint32]
        L.tfb_reader_tensor_block_formats.restype = C.c_long
        L.tfb_reader_tensor_block_formats.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_long]
        _LIB = L
    return _LIB


# ---------------------------------------------------------------------------------------------- registry
def format_name(fmt: int) -> str:
    n = lib().tfb_format_name(fmt)
    return n.decode() if n else "unknown"


def parse_format(name: str) -> int:
    return lib().tfb_format_parse(name.encode())


def format_bpw(fmt: int) -> float:
    return lib().tfb_format_bpw(fmt)


def is_wire_exact(fmt: int) -> bool:
    return bool(lib().tfb_format_is_wire_exact(fmt))


def claimed_bytes(fmt: int, n: int) -> int:
    return lib().tfb_block_claimed_bytes(fmt, n)


def all_formats():
    return [(i, format_name(i), format_bpw(i)) for i in range(FORMAT_COUNT)]


# ---------------------------------------------------------------------------------------------- blocks
def quantize_block(fmt: int, w) -> bytes:
    a = np.ascontiguousarray(np.asarray(w, dtype=np.float32))
    cap = max(claimed_bytes(fmt, a.size), a.size * 4) + 16
    buf = (C.c_uint8 * cap)()
    got = lib().tfb_quantize_block(fmt, a.ctypes.data, a.size, buf, cap)
    if got < 0:
        raise ValueError(f"quantize_block({format_name(fmt)}, n={a.size}) failed")
    return bytes(buf[:got])


def dequantize_block(fmt: int, payload: bytes, n: int) -> np.ndarray:
    out = np.zeros(n, dtype=np.float32)
    b = (C.c_uint8 * max(1, len(payload))).from_buffer_copy(payload or b"\0")
    lib().tfb_dequantize_block(fmt, b, len(payload), None, 0, n, out.ctypes.data)
    return out


def sha256(data: bytes) -> bytes:
    out = (C.c_uint8 * 32)()
    lib().tfb_sha256(data, len(data), out)
    return bytes(out)


# ---------------------------------------------------------------------------------------------- container
class QuantReader:
    def __init__(self, path):
        self._h = lib().tfb_reader_open(str(path).encode())
        if not self._h or not lib().tfb_reader_valid(self._h):
            if self._h:
                lib().tfb_reader_close(self._h)
                self._h = None
            raise ValueError(f"{path}: not a valid .quant container")

    def close(self):
        if self._h:
            lib().tfb_reader_close(self._h)
            self._h = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def version(self):
        return lib().tfb_reader_version(self._h)

    def config_bytes(self) -> bytes:
        n = lib().tfb_reader_config(self._h, None, 0)
        buf = (C.c_uint8 * max(1, n))()
        lib().tfb_reader_config(self._h, buf, n)
        return bytes(buf[:n])

    def tensor_names(self):
        return [lib().tfb_reader_tensor_name(self._h, i).decode() for i in range(lib().tfb_reader_num_tensors(self._h))]

    def num_blocks(self):
        return lib().tfb_reader_num_blocks(self._h)

    def tensor_format(self, name) -> int:
        return lib().tfb_reader_tensor_format(self._h, name.encode())

    def block_formats(self, name):
        """Format id of every block of a tensor."""
        n = lib().tfb_reader_tensor_block_formats(self._h, name.encode(), None, 0)
        if n < 0:
            raise KeyError(name)
        out = np.empty(max(1, n), dtype=np.uint8)
        lib().tfb_reader_tensor_block_formats(self._h, name.encode(), out.ctypes.data, n)
        return out[:n]

    # ---- block-level verbs of the reference reader (include/quant/quant_format.h:90-140)
    def valid(self) -> bool:
        return bool(self._h) and bool(lib().tfb_reader_valid(self._h))

    def header(self) -> dict:
        """{magic, version, flags, config_size} of the 16-byte file header."""
        return {"magic": "QUA1", "version": int(self.version), "flags": int(lib().tfb_reader_flags(self._h)),
                "config_size": int(lib().tfb_reader_config(self._h, None, 0))}

    def _block_info(self, b: int):
        info = (C.c_uint32 * 6)()
        if lib().tfb_reader_block_info(self._h, int(b), info) != 0:
            raise IndexError(f"block {b} of {self.num_blocks()}")
        return [int(v) for v in info]

    # ---- fail-closed block addressing (reference: QUANTReader, include/quant/quant_format.h:85-124): a block id from an
    # untrusted file never raises here; the caller checks the sentinel
    INVALID_FORMAT = 0xFF

    def block_offset(self, b: int) -> int:
        """Byte offset of block ``b``'s record in the file; -1 when there is no such block."""
        return int(lib().tfb_reader_block_offset(self._h, int(b))) if 0 <= int(b) < (1 << 32) else -1

    def range_ok(self, start: int, count: int) -> bool:
        """Whether blocks [start, start + count) all exist."""
        return start >= 0 and count >= 0 and start + count <= self.num_blocks()

    def format_entry(self, b: int):
        """(block_id, format byte, codebook bytes) of the table entry of block ``b``; the format byte is 0xFF (no format has
        that code) for a block that does not exist."""
        if not self.range_ok(int(b), 1):
            return (int(b), self.INVALID_FORMAT, 0)
        return tuple(self._block_info(b)[:3])

    def block_ptr(self, b: int):
        """The whole stored record of block ``b`` (u32 weights, u32 codebook bytes, codebook, u32 index bytes, indices);
        None when there is no such block."""
        if not self.range_ok(int(b), 1):
            return None
        blk = self.read_block(b)
        import struct
        return struct.pack("<II", blk.num_weights, len(blk.codebook)) + blk.codebook + struct.pack("<I", len(blk.indices)) + blk.indices

    def read_config(self) -> bytes:
        return self.config_bytes()

    def read_format_table(self):
        """[(block_id, format byte, codebook bytes)] as stored in the table, one entry per block."""
        return [tuple(self._block_info(b)[:3]) for b in range(self.num_blocks())]

    def block_sizes(self, b: int):
        """(num_weights, codebook bytes, index bytes) of block ``b``."""
        i = self._block_info(b)
        return i[3], i[4], i[5]

    def read_block(self, b: int) -> "BlockData":
        """Block ``b`` as stored: its format, weight count and the raw codebook / index bytes."""
        i = self._block_info(b)
        cb, ib = (C.c_uint8 * max(1, i[4]))(), (C.c_uint8 * max(1, i[5]))()
        lib().tfb_reader_block_payload(self._h, int(b), cb, ib)
        return BlockData(i[1], i[3], bytes(ib[:i[5]]), bytes(cb[:i[4]]))

    def decode_block(self, b: int) -> np.ndarray:
        """The weights of block ``b`` alone."""
        n = self._block_info(b)[3]
        out = np.empty(max(1, n), dtype=np.float32)
        got = lib().tfb_reader_decode_block(self._h, int(b), out.ctypes.data, n)
        if got != n:
            raise ValueError(f"block {b}: cannot be decoded ({got})")
        return out[:n]

    def tensor_blocks(self, name: str):
        """(first block, number of blocks) of a tensor."""
        s, c = C.c_uint32(), C.c_uint32()
        if lib().tfb_reader_tensor_range(self._h, name.encode(), C.byref(s), C.byref(c)) != 0:
            raise KeyError(name)
        return int(s.value), int(c.value)

    def tensor_formats(self, name: str):
        """Format byte of every block of a tensor (the reference's name for ``block_formats``)."""
        return self.block_formats(name).tolist()

    def read_tensor(self, name) -> torch.Tensor:
        n = lib().tfb_reader_tensor_numel(self._h, name.encode())
        if n < 0:
            raise KeyError(name)
        out = np.empty(n, dtype=np.float32)
        got = lib().tfb_reader_read_tensor(self._h, name.encode(), out.ctypes.data, n)
        if got == -2:
            raise ValueError(f"{name}: stored in format {format_name(self.tensor_format(name))}, whose block stream from another "
                             "encoder this library cannot decode (only the formats `quant_format_list` marks wire-exact "
                             "interchange with files written elsewhere); re-export the file in a wire-exact format")
        if got != n:
            raise ValueError(f"{name}: corrupt blocks")
        return torch.from_numpy(out)


class BlockData:
    """One stored block: format byte, number of weights, index bytes (the block stream) and codebook bytes."""

    def __init__(self, format: int, num_weights: int, indices: bytes = b"", codebook: bytes = b""):
        self.format, self.num_weights, self.indices, self.codebook = int(format), int(num_weights), bytes(indices), bytes(codebook)

    @classmethod
    def encode(cls, fmt, weights) -> "BlockData":
        """Quantise a block of weights into ``fmt``."""
        f = parse_format(fmt) if isinstance(fmt, str) else int(fmt)
        a = np.ascontiguousarray(np.asarray(weights, dtype=np.float32).reshape(-1))
        return cls(f, a.size, quantize_block(f, a))

    def decode(self) -> np.ndarray:
        return dequantize_block(self.format, self.indices, self.num_weights)


class QuantWriter:
    """Two ways to write a container.  ``add_tensor`` / ``add_tensor_mixed`` + ``close`` encode tensors and lay the file
    out themselves.  The streaming verbs ``write_header`` / ``write_format_table`` / ``write_tensor_table`` /
    ``write_block`` / ``write_raw`` (reference: QUANTWriter, include/quant/quant_format.h:34-88) append to the file in the
    order they are called, for callers that build the tables themselves or copy blocks between files without decoding;
    a file is readable when the order is header, format table, tensor table, blocks."""

    def __init__(self, path, config: bytes = b"", version: int = 1, flags: int = 0):
        self.path = str(path)
        self._stream = None
        self._cfg = (config, version, flags)
        self._h = None

    def _handle(self):
        if self._stream is not None:
            raise RuntimeError("this writer is in streaming mode (write_header was called)")
        if self._h is None:
            config, version, flags = self._cfg
            self._h = lib().tfb_writer_open(self.path.encode(), version, flags, config, len(config))
        return self._h

    # ---- streaming verbs
    def _file(self):
        if self._h is not None:
            raise RuntimeError("this writer already holds encoded tensors (add_tensor was called)")
        if self._stream is None:
            self._stream = open(self.path, "wb")
            self._names = []
        return self._stream

    def write_header(self, version: int = 1, flags: int = 0, config: bytes = b""):
        import struct
        self._file().write(b"QUA1" + struct.pack("<III", version, flags, len(config)) + bytes(config))

    def write_format_table(self, entries):
        """``entries``: (block_id, format byte, codebook bytes) per block."""
        import struct
        f = self._file()
        f.write(struct.pack("<I", len(entries)))
        for bid, fmt, cb in entries:
            f.write(struct.pack("<IBI", bid, fmt, cb))

    def write_tensor_table(self, entries, names):
        """``entries``: (first block, number of blocks) per tensor, ``names`` in the same order."""
        import struct
        f = self._file()
        f.write(struct.pack("<I", len(entries)))
        for (start, count), name in zip(entries, names):
            nb = name.encode()
            f.write(struct.pack("<H", len(nb)) + nb + struct.pack("<II", start, count))
        self._names = list(names)

    def write_block(self, block: "BlockData"):
        import struct
        self._file().write(struct.pack("<II", block.num_weights, len(block.codebook)) + block.codebook +
                           struct.pack("<I", len(block.indices)) + block.indices)

    def write_raw(self, data: bytes):
        self._file().write(bytes(data))

    def write_dedup(self, payload: bytes, store: "DedupStore") -> str:
        """Put ``payload`` into a content-addressed store next to the file and return its key (identical payloads are
        stored once)."""
        return store.write_dedup(payload)

    def add_tensor(self, name: str, t: torch.Tensor, fmt: int = Q_32, block: int | None = None):
        a = t.detach().float().cpu().contiguous().numpy().reshape(-1)
        if block is None:
            block = 32768 if fmt == Q_32 else 256
        if lib().tfb_writer_add_tensor(self._handle(), name.encode(), a.ctypes.data, a.size, fmt, block) != 0:
            raise ValueError(f"add_tensor({name}) failed")

    def add_tensor_mixed(self, name: str, t: torch.Tensor, fmts, block: int = 256):
        """One format per ``block`` weights (a FormatPlan's assignment)."""
        a = t.detach().float().cpu().contiguous().numpy().reshape(-1)
        f = np.ascontiguousarray(np.asarray(fmts, dtype=np.uint8))
        if lib().tfb_writer_add_tensor_mixed(self._handle(), name.encode(), a.ctypes.data, a.size, f.ctypes.data, f.size, block) != 0:
            raise ValueError(f"add_tensor_mixed({name}) failed")

    def close(self, write_idx=True):
        if self._stream is not None:
            self._stream.close()
            self._stream = None
            if write_idx and self._names:
                import struct
                with open(self.path + ".idx", "wb") as g:
                    g.write(IDX_MAGICS[0] + struct.pack("<II", 1, len(self._names)))
                    for name in self._names:
                        nb = name.encode()
                        g.write(struct.pack("<H", len(nb)) + nb + sha256(nb))
            return
        if self._h is None and self._cfg is not None:
            self._handle()                     # a writer closed without tensors still writes a valid, empty container
        h, self._h = self._h, None
        if h and lib().tfb_writer_close(h, int(write_idx)) != 0:
            raise IOError("writing .quant failed")


def save_model(model, path, fmt: int | str = Q_32, per_layer: dict | None = None):
    """DenseModel / MoEModel -> .quant with the reference tensor names.  ``per_layer`` maps a name
    substring to a format (the ``--per-layer name=fmt`` rule of quant_quantize)."""
    if isinstance(fmt, str):
        fmt = parse_format(fmt)
    w = QuantWriter(path, model.cfg.to_bytes())
    for name, t in model.named_tensors():
        f = fmt
        for key, pf in (per_layer or {}).items():
            if key in name:
                f = parse_format(pf) if isinstance(pf, str) else pf
        if t.dim() < 2 and f != Q_32:
            f = Q_32   # norms and biases stay exact
        w.add_tensor(name, t, f)
    w.close()


def load_state(path):
    """(config bytes, {name: fp32 tensor}) of a .quant file."""
    with QuantReader(path) as r:
        return r.config_bytes(), {n: r.read_tensor(n) for n in r.tensor_names()}


def load_model(path, device="cpu", dtype=torch.float32, model_cls=None, strict=True, **cfg_extra):
    """Rebuild a DenseModel from a .quant file (shapes come from the config; names must match)."""
    from ..models.config import TransformerConfig
    from ..models.dense import DenseModel
    raw, tensors = load_state(path)
    cfg = TransformerConfig.from_bytes(raw, **cfg_extra)
    if "lm_head.weight" not in tensors:
        cfg.tie_embeddings = True
    model = (model_cls or DenseModel)(cfg, device=device, dtype=dtype, seed=None)
    with torch.no_grad():
        for name, dst in model.named_tensors():
            if name not in tensors:
                if strict:
                    raise KeyError(f"{path}: tensor {name} missing")
                continue
            src = tensors[name]
            if src.numel() != dst.numel():
                raise ValueError(f"{name}: {src.numel()} weights in file, {dst.numel()} expected")
            dst.copy_(src.view(dst.shape).to(dst.dtype))
    return model


# ------------------------------------------------------------------------------------------------ index side-car, dedup store
IDX_MAGICS = (b"TransFormers-FusionIDX", b"TransCenderIDX", b"InNovaIDX")      # current, then the two legacy spellings


def read_index(path: str):
    """Parses ``<model>.quant.idx``: magic | u32 version | u32 n | per tensor {u16 len, name, sha256(name)}.  Accepts the
    current magic and both legacy ones.  Returns (version, [(name, digest)])."""
    import struct
    data = open(path, "rb").read()
    magic = next((m for m in IDX_MAGICS if data.startswith(m)), None)
    if magic is None:
        raise ValueError(f"{path}: not a tensor index")
    off = len(magic)
    ver, n = struct.unpack_from("<II", data, off)
    off += 8
    out = []
    for _ in range(n):
        (ln,) = struct.unpack_from("<H", data, off)
        off += 2
        name = data[off:off + ln].decode("utf-8")
        off += ln
        out.append((name, data[off:off + 32]))
        off += 32
    if off != len(data):
        raise ValueError(f"{path}: {len(data) - off} trailing bytes")
    return ver, out


def verify_index(quant_path: str) -> bool:
    """The side-car lists exactly the tensors of the container, in order, with sha256(name) digests."""
    _, entries = read_index(quant_path + ".idx")
    with QuantReader(quant_path) as r:
        names = r.tensor_names()
    return [n for n, _ in entries] == list(names) and all(sha256(n.encode()) == d for n, d in entries)


class DedupStore:
    """Content-addressed blob store: ``write_dedup`` keeps one copy of identical payloads (tied embeddings, repeated
    experts after upcycling, shared codebooks) under ``<dir>/<sha256 hex>`` and returns the digest.
    Reference counterpart: QUANTWriter::write_dedup (sha256 content addressing, src/codec/quant_format.cpp)."""

    def __init__(self, directory: str):
        import os
        self.dir = directory
        os.makedirs(directory, exist_ok=True)
        self.writes = self.hits = 0

    def write_dedup(self, payload: bytes) -> str:
        import os
        key = sha256(payload).hex()
        p = os.path.join(self.dir, key)
        if os.path.exists(p):
            self.hits += 1
        else:
            tmp = p + ".tmp"
            with open(tmp, "wb") as f:
                f.write(payload)
            os.replace(tmp, p)
            self.writes += 1
        return key

    def read(self, key: str) -> bytes:
        import os
        data = open(os.path.join(self.dir, key), "rb").read()
        if sha256(data).hex() != key:
            raise ValueError(f"blob {key} is corrupt")
        return data

    def write_tensor(self, t: torch.Tensor) -> str:
        return self.write_dedup(t.detach().contiguous().cpu().numpy().tobytes())
