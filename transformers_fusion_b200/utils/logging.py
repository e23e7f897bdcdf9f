"""Run logging: ``Logger`` (levels, optional file), ``EventWriter`` (TensorBoard event files written without any
dependency: TFRecord framing with masked CRC32C around hand-encoded Event/Summary protobufs), ``WandBLogger`` (a
``metrics.json`` line log per run), and ``AppConfig`` (JSON configuration with dotted-path access and validation).

Reference counterparts: EventWriter / WandBLogger (include/quant/log_writer.h), Logger and AppConfig
(include/quant/production.h:220-284)."""
from __future__ import annotations

import json
import os
import struct
import sys
import threading
import time
from typing import Any, Dict, Optional


class Logger:
    LEVELS = {"debug": 10, "info": 20, "warn": 30, "error": 40}

    def __init__(self, level="info", path: Optional[str] = None, stream=sys.stderr):
        self.level = self.LEVELS[level]
        self.file = open(path, "a") if path else None
        self.stream, self.lock = stream, threading.Lock()

    DEBUG, INFO, WARN, ERROR = "debug", "info", "warn", "error"
    _instance: Optional["Logger"] = None

    @classmethod
    def instance(cls) -> "Logger":
        """The process-wide logger (created on first use at level info, writing to stderr)."""
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def set_file(self, path: Optional[str]):
        """Also append every line to ``path`` (None stops writing to a file)."""
        with self.lock:
            if self.file:
                self.file.close()
            self.file = open(path, "a") if path else None

    def set_level(self, level):
        self.level = self.LEVELS[self._name(level)]

    @staticmethod
    def _name(level):
        """Level names, or the reference's numeric levels 0..3 (include/quant/production.h: Logger::Level)."""
        return ("debug", "info", "warn", "error")[level] if isinstance(level, int) else str(level).lower()

    def log(self, level, msg):
        level = self._name(level)
        if self.LEVELS[level] < self.level:
            return
        line = f"{time.strftime('%Y-%m-%d %H:%M:%S')} [{level.upper()}] {msg}\n"
        with self.lock:
            if self.stream:
                self.stream.write(line)
            if self.file:
                self.file.write(line)
                self.file.flush()

    def debug(self, m): self.log("debug", m)
    def info(self, m): self.log("info", m)
    def warn(self, m): self.log("warn", m)
    def error(self, m): self.log("error", m)

    def close(self):
        if self.file:
            self.file.close()
            self.file = None


# ---- CRC32C (Castagnoli), table driven -----------------------------------------------------------------------
_CRC_TABLE = []
for _i in range(256):
    _c = _i
    for _ in range(8):
        _c = (_c >> 1) ^ 0x82F63B78 if _c & 1 else _c >> 1
    _CRC_TABLE.append(_c)


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


class EventWriter:
    """Scalars into ``<logdir>/events.out.tfevents.<time>.<host>`` readable by TensorBoard."""

    def __init__(self, logdir: str):
        os.makedirs(logdir, exist_ok=True)
        self.path = os.path.join(logdir, f"events.out.tfevents.{int(time.time())}.{os.uname().nodename}")
        self.f = open(self.path, "ab")
        self.lock = threading.Lock()
        self._record(_field(1, 1, struct.pack("<d", time.time())) + _field(3, 2, _varint(len(b"brain.Event:2")) + b"brain.Event:2"))

    def _record(self, event: bytes):
        hdr = struct.pack("<Q", len(event))
        self.f.write(hdr + struct.pack("<I", _masked_crc(hdr)) + event + struct.pack("<I", _masked_crc(event)))

    def write_scalar(self, tag: str, value: float, step: int, wall_time: Optional[float] = None):
        t = tag.encode()
        val = _field(1, 2, _varint(len(t)) + t) + _field(2, 5, struct.pack("<f", float(value)))          # Summary.Value
        summ = _field(1, 2, _varint(len(val)) + val)                                                       # Summary
        ev = _field(1, 1, struct.pack("<d", wall_time or time.time())) + _field(2, 0, _varint(int(step))) + \
            _field(5, 2, _varint(len(summ)) + summ)                                                        # Event
        with self.lock:
            self._record(ev)

    def write_scalars(self, metrics, step: int):
        for k in ("loss", "perplexity", "val_loss", "learning_rate", "grad_norm", "tokens_per_sec"):
            if hasattr(metrics, k):
                self.write_scalar(f"train/{k}", getattr(metrics, k), step)

    def flush(self):
        with self.lock:
            self.f.flush()

    def close(self):
        self.flush()
        self.f.close()


def read_event_scalars(path):
    """[(step, tag, value)] from an event file (verifies the record checksums); used by tests and tools."""
    out = []
    data = open(path, "rb").read()
    o = 0

    def parse(buf):
        i, fields = 0, []
        while i < len(buf):
            key, sh = 0, 0
            while True:
                b = buf[i]; i += 1
                key |= (b & 0x7F) << sh; sh += 7
                if not b & 0x80:
                    break
            num, wire = key >> 3, key & 7
            if wire == 0:
                v, sh = 0, 0
                while True:
                    b = buf[i]; i += 1
                    v |= (b & 0x7F) << sh; sh += 7
                    if not b & 0x80:
                        break
                fields.append((num, v))
            elif wire == 1:
                fields.append((num, buf[i:i + 8])); i += 8
            elif wire == 5:
                fields.append((num, buf[i:i + 4])); i += 4
            else:
                ln, sh = 0, 0
                while True:
                    b = buf[i]; i += 1
                    ln |= (b & 0x7F) << sh; sh += 7
                    if not b & 0x80:
                        break
                fields.append((num, buf[i:i + ln])); i += ln
        return fields
    while o + 12 <= len(data):
        (n,) = struct.unpack_from("<Q", data, o)
        if struct.unpack_from("<I", data, o + 8)[0] != _masked_crc(data[o:o + 8]):
            raise ValueError("bad length checksum")
        ev = data[o + 12:o + 12 + n]
        if struct.unpack_from("<I", data, o + 12 + n)[0] != _masked_crc(ev):
            raise ValueError("bad record checksum")
        o += 16 + n
        f = dict(parse(ev))
        if 5 in f:
            for num, val in parse(f[5]):
                vf = dict(parse(val))
                out.append((f.get(2, 0), vf[1].decode(), struct.unpack("<f", vf[2])[0]))
    return out


class WandBLogger:
    def __init__(self, project: str, run_name: str = "", root: str = "."):
        self.run_name = run_name or time.strftime("run-%Y%m%d-%H%M%S")
        d = os.path.join(root, "wandb", project, self.run_name)
        os.makedirs(d, exist_ok=True)
        self.path = os.path.join(d, "metrics.json")
        self.f = open(self.path, "a")
        self.lock = threading.Lock()

    def log(self, key: str, value: float, step: int):
        with self.lock:
            self.f.write(json.dumps({"_step": int(step), "_timestamp": time.time(), key: float(value)}) + "\n")

    def log_metrics(self, metrics, step: int):
        row = {"_step": int(step), "_timestamp": time.time()}
        for k in ("loss", "perplexity", "val_loss", "learning_rate", "grad_norm", "tokens_per_sec", "epoch"):
            if hasattr(metrics, k):
                row[k] = float(getattr(metrics, k))
        with self.lock:
            self.f.write(json.dumps(row) + "\n")

    def flush(self):
        with self.lock:
            self.f.flush()

    def close(self):
        self.flush()
        self.f.close()


class AppConfig:
    """JSON configuration with ``get("server.port", default)`` / ``set`` / ``save`` / ``validate``."""

    def __init__(self, path: Optional[str] = None, data: Optional[dict] = None):
        self.path = path
        self.data: Dict[str, Any] = data or {}
        if path and os.path.exists(path):
            with open(path) as f:
                self.data = json.load(f)

    def get(self, dotted: str, default=None):
        cur = self.data
        for part in dotted.split("."):
            if not isinstance(cur, dict) or part not in cur:
                return default
            cur = cur[part]
        return cur

    # ---- typed getters of the reference (include/quant/production.h: AppConfig)
    def get_int(self, key: str, default: int = 0) -> int:
        v = self.get(key)
        try:
            return int(v) if v is not None and not isinstance(v, (dict, list)) else default
        except (TypeError, ValueError):
            return default

    def get_float(self, key: str, default: float = 0.0) -> float:
        v = self.get(key)
        try:
            return float(v) if v is not None and not isinstance(v, (dict, list, bool)) else default
        except (TypeError, ValueError):
            return default

    def get_string(self, key: str, default: str = "") -> str:
        v = self.get(key)
        return default if v is None or isinstance(v, (dict, list)) else (str(v).lower() if isinstance(v, bool) else str(v))

    def to_json(self, indent: int = 2) -> str:
        return json.dumps(self.data, indent=indent, sort_keys=True)

    def set(self, dotted: str, value):
        if isinstance(value, str):                       # text from a command line becomes the value it spells
            low = value.strip().lower()
            if low in ("true", "false"):
                value = low == "true"
            else:
                try:
                    value = int(value)
                except ValueError:
                    try:
                        value = float(value)
                    except ValueError:
                        pass
        cur = self.data
        parts = dotted.split(".")
        for part in parts[:-1]:
            cur = cur.setdefault(part, {})
            if not isinstance(cur, dict):
                raise ValueError(f"{dotted}: '{part}' is not an object")
        cur[parts[-1]] = value

    def save(self, path: Optional[str] = None):
        p = path or self.path
        tmp = p + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.data, f, indent=2, sort_keys=True)
        os.replace(tmp, p)

    def validate(self, schema: Dict[str, type]):
        """``schema`` maps dotted paths to required types; returns the list of problems (empty = valid)."""
        errs = []
        for k, t in schema.items():
            v = self.get(k)
            if v is None:
                errs.append(f"{k}: missing")
            elif not isinstance(v, t) or (t is int and isinstance(v, bool)):
                errs.append(f"{k}: expected {t.__name__}, got {type(v).__name__}")
        return errs
