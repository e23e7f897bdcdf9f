"""Core value types and thread-safety helpers.

Types: DType (element kinds of the codec and the kernels), Shape (rank <= 8), Status (ok / message), Config (process-wide
defaults), quant_check.  Thread-safety: single-producer single-consumer ring, readers-writer mutex, atomic float
accumulator, spin lock, named counters.  Python threads share the GIL, so these exist for API parity and for code that
hands work between the server's worker threads; the device side has its own (mbarrier, flag) primitives.

Reference counterparts: include/quant/types.h:289-314 (DType, Shape, Status, Config, QUANT_CHECK),
include/quant/thread_safety.h:28-255 (SPSCQueue, SharedMutex, AtomicFloat, SpinLock, ThreadSafeCounter)."""
from __future__ import annotations

import enum
import threading
from dataclasses import dataclass
from typing import Generic, List, Optional, Tuple, TypeVar

T = TypeVar("T")


class DType(enum.IntEnum):
    I64 = 0
    I32 = 1
    U8 = 2
    U4 = 3
    U16 = 4
    F16 = 5
    F32 = 6
    BF16 = 7       # additions of this framework: the compute type and the two 8-bit float storage types
    E4M3 = 8
    E5M2 = 9

    @property
    def bits(self) -> int:
        return {0: 64, 1: 32, 2: 8, 3: 4, 4: 16, 5: 16, 6: 32, 7: 16, 8: 8, 9: 8}[int(self)]

    def torch(self):
        import torch
        return {0: torch.int64, 1: torch.int32, 2: torch.uint8, 3: torch.uint8, 4: torch.int16, 5: torch.float16, 6: torch.float32,
                7: torch.bfloat16, 8: torch.float8_e4m3fn, 9: torch.float8_e5m2}[int(self)]


class Shape(tuple):
    """Immutable dimension list of rank <= 8."""
    MAX_RANK = 8

    def __new__(cls, *dims):
        if len(dims) == 1 and isinstance(dims[0], (tuple, list)):
            dims = tuple(dims[0])
        if len(dims) > cls.MAX_RANK:
            raise ValueError(f"rank {len(dims)} exceeds {cls.MAX_RANK}")
        if any(int(d) < 0 for d in dims):
            raise ValueError("negative dimension")
        return super().__new__(cls, (int(d) for d in dims))

    @property
    def rank(self) -> int: return len(self)

    def to_string(self) -> str:
        return "[" + ", ".join(str(d) for d in self) + "]"

    def numel(self) -> int:
        n = 1
        for d in self:
            n *= d
        return n

    def strides(self) -> Tuple[int, ...]:
        out, s = [], 1
        for d in reversed(self):
            out.append(s)
            s *= d
        return tuple(reversed(out))


@dataclass(frozen=True)
class Status:
    ok: bool = True
    message: str = ""

    @staticmethod
    def OK() -> "Status": return Status(True, "")

    @staticmethod
    def error(msg: str) -> "Status": return Status(False, msg)

    @staticmethod
    def success() -> "Status": return Status(True, "")

    @property
    def msg(self) -> str: return self.message

    def __bool__(self) -> bool: return self.ok


@dataclass
class Config:
    num_threads: int = 0          # 0 = all cores
    seed: int = 42
    pool_bytes: int = 64 << 20


def quant_check(cond, msg: str = "check failed"):
    if not cond:
        raise RuntimeError(f"QUANT_CHECK: {msg}")


# ------------------------------------------------------------------------------------------------ thread safety
class SPSCQueue(Generic[T]):
    """Bounded ring for one producer thread and one consumer thread.  ``push`` / ``pop`` never block: they report
    full / empty.  Head and tail are only written by their own side."""

    def __init__(self, capacity: int):
        if capacity < 1:
            raise ValueError("capacity must be positive")
        self._buf: List[Optional[T]] = [None] * (capacity + 1)
        self._head = 0          # next slot to pop   (consumer)
        self._tail = 0          # next slot to push  (producer)

    def push(self, item: T) -> bool:
        nxt = (self._tail + 1) % len(self._buf)
        if nxt == self._head:
            return False
        self._buf[self._tail] = item
        self._tail = nxt
        return True

    def pop(self) -> Optional[T]:
        if self._head == self._tail:
            return None
        item, self._buf[self._head] = self._buf[self._head], None
        self._head = (self._head + 1) % len(self._buf)
        return item

    def __len__(self) -> int:
        return (self._tail - self._head) % len(self._buf)

    @property
    def capacity(self) -> int: return len(self._buf) - 1
    def empty(self) -> bool: return self._head == self._tail


class SharedMutex:
    """Readers-writer lock: any number of shared holders or one exclusive holder; waiting writers block new readers."""

    def __init__(self):
        self._cv = threading.Condition()
        self._readers, self._writer, self._waiting_writers = 0, False, 0

    def lock_shared(self):
        with self._cv:
            while self._writer or self._waiting_writers:
                self._cv.wait()
            self._readers += 1

    def unlock_shared(self):
        with self._cv:
            self._readers -= 1
            if self._readers == 0:
                self._cv.notify_all()

    def lock(self):
        with self._cv:
            self._waiting_writers += 1
            while self._writer or self._readers:
                self._cv.wait()
            self._waiting_writers -= 1
            self._writer = True

    def unlock(self):
        with self._cv:
            self._writer = False
            self._cv.notify_all()

    def try_lock(self) -> bool:
        """Take the exclusive lock only if nobody holds the lock in either mode; never waits."""
        with self._cv:
            if self._writer or self._readers:
                return False
            self._writer = True
            return True

    def try_lock_shared(self) -> bool:
        with self._cv:
            if self._writer or self._waiting_writers:
                return False
            self._readers += 1
            return True

    def shared(self):
        return _Guard(self.lock_shared, self.unlock_shared)

    def unique(self):
        return _Guard(self.lock, self.unlock)


class _Guard:
    def __init__(self, acquire, release):
        self._a, self._r = acquire, release

    def __enter__(self):
        self._a()
        return self

    def __exit__(self, *exc):
        self._r()
        return False


class AtomicFloat:
    def __init__(self, value: float = 0.0):
        self._v, self._l = float(value), threading.Lock()

    def load(self) -> float:
        with self._l:
            return self._v

    def store(self, v: float):
        with self._l:
            self._v = float(v)

    def fetch_add(self, d: float) -> float:
        with self._l:
            old = self._v
            self._v += d
            return old

    def fetch_max(self, v: float) -> float:
        with self._l:
            old = self._v
            self._v = max(self._v, v)
            return old

    def compare_exchange(self, expected: float, desired: float) -> bool:
        with self._l:
            if self._v == expected:
                self._v = float(desired)
                return True
            return False


class SpinLock:
    """Non-blocking acquire in a loop (short critical sections only)."""

    def __init__(self):
        self._l = threading.Lock()

    def lock(self):
        while not self._l.acquire(blocking=False):
            pass

    def try_lock(self) -> bool: return self._l.acquire(blocking=False)
    def unlock(self): self._l.release()
    def __enter__(self):
        self.lock()
        return self

    def __exit__(self, *exc):
        self.unlock()
        return False


class ThreadSafeCounter:
    def __init__(self):
        self._c, self._l = {}, threading.Lock()

    def increment(self, name: str = "", by: int = 1) -> int:
        with self._l:
            self._c[name] = self._c.get(name, 0) + by
            return self._c[name]

    def get(self, name: str = "") -> int:
        with self._l:
            return self._c.get(name, 0)

    def reset(self, name: Optional[str] = None):
        with self._l:
            if name is None:
                self._c.clear()
            else:
                self._c.pop(name, None)

    def snapshot(self) -> dict:
        with self._l:
            return dict(self._c)

    def add(self, n: int = 1, name: str = "") -> int:
        return self.increment(name, n)

    def total(self) -> int:
        with self._l:
            return sum(self._c.values())


# ------------------------------------------------------------------------------------------------ files and JSON values
class MappedFile:
    """Read-only memory map of a file with bounds-checked slices (reference MappedFile, src/codec/quant_format.cpp:624-721)."""

    def __init__(self, path: str):
        import mmap
        self.path = path
        self._f = open(path, "rb")
        self.size = self._f.seek(0, 2)
        self._m = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if self.size else None

    def valid(self) -> bool: return self._f is not None

    def read(self, offset: int, n: int) -> bytes:
        if offset < 0 or n < 0 or offset + n > self.size:
            raise ValueError(f"read of [{offset}, {offset + n}) outside a file of {self.size} bytes")
        return bytes(self._m[offset:offset + n]) if n else b""

    def view(self) -> memoryview:
        return memoryview(self._m) if self._m is not None else memoryview(b"")

    def close(self):
        if self._m is not None:
            self._m.close()
        if self._f is not None:
            self._f.close()
        self._m = self._f = None

    def __enter__(self): return self
    def __exit__(self, *exc):
        self.close()
        return False


class JsonValue:
    """Parsed JSON with dotted-path access and typed getters that fall back to a default instead of raising
    (reference JsonValue, src/server/json_parser.cpp)."""

    def __init__(self, value=None):
        self.value = value

    @staticmethod
    def parse(text: str) -> "JsonValue":
        import json
        return JsonValue(json.loads(text))

    def get(self, path: str, default=None):
        cur = self.value
        for part in path.split(".") if path else []:
            if isinstance(cur, dict) and part in cur:
                cur = cur[part]
            elif isinstance(cur, list) and part.lstrip("-").isdigit() and -len(cur) <= int(part) < len(cur):
                cur = cur[int(part)]
            else:
                return default
        return cur

    def get_int(self, path, default=0):
        v = self.get(path, default)
        return int(v) if isinstance(v, (int, float)) and not isinstance(v, bool) else default

    def get_float(self, path, default=0.0):
        v = self.get(path, default)
        return float(v) if isinstance(v, (int, float)) and not isinstance(v, bool) else default

    def get_str(self, path, default=""):
        v = self.get(path, default)
        return v if isinstance(v, str) else default

    def get_bool(self, path, default=False):
        v = self.get(path, default)
        return v if isinstance(v, bool) else default

    def is_object(self): return isinstance(self.value, dict)
    def is_array(self): return isinstance(self.value, list)

    # ---- node-level accessors of the reference (include/quant/json_parser.h): a JsonValue wraps ONE node
    NUL, BOOL, INT, FLOAT, STRING, ARRAY, OBJECT = range(7)

    @property
    def type(self) -> int:
        v = self.value
        return (self.NUL if v is None else self.BOOL if isinstance(v, bool) else self.INT if isinstance(v, int) else
                self.FLOAT if isinstance(v, float) else self.STRING if isinstance(v, str) else self.ARRAY if isinstance(v, list) else self.OBJECT)

    def is_null(self): return self.value is None
    def is_bool(self): return isinstance(self.value, bool)
    def is_number(self): return isinstance(self.value, (int, float)) and not isinstance(self.value, bool)
    def is_string(self): return isinstance(self.value, str)

    def as_bool(self) -> bool: return self.value if isinstance(self.value, bool) else False
    def as_int(self) -> int: return int(self.value) if self.is_number() else 0
    def as_float(self) -> float: return float(self.value) if self.is_number() else 0.0
    def as_string(self) -> str: return self.value if isinstance(self.value, str) else ""

    def _checked(self, ok: bool, what: str):
        if not ok:
            raise TypeError(f"JsonValue: not {what}")
        return self.value

    def as_bool_checked(self) -> bool: return self._checked(self.is_bool(), "a bool")
    def as_int_checked(self) -> int: return self._checked(self.type == self.INT, "an int")
    def as_float_checked(self) -> float: return float(self._checked(self.is_number(), "a number"))
    def as_string_checked(self) -> str: return self._checked(self.is_string(), "a string")

    @property
    def bool_val(self): return self.as_bool()
    @property
    def int_val(self): return self.as_int()
    @property
    def float_val(self): return self.as_float()
    @property
    def str_val(self): return self.as_string()
    @property
    def arr(self): return [JsonValue(v) for v in self.value] if isinstance(self.value, list) else []
    @property
    def obj(self): return {k: JsonValue(v) for k, v in self.value.items()} if isinstance(self.value, dict) else {}
    arr_val, obj_val = arr, obj

    def has(self, key: str) -> bool: return isinstance(self.value, dict) and key in self.value

    def __getitem__(self, key) -> "JsonValue":
        """Object member (a null node when absent) or array element (IndexError when out of range)."""
        if isinstance(key, str):
            return JsonValue(self.value.get(key) if isinstance(self.value, dict) else None)
        if not isinstance(self.value, list) or not -len(self.value) <= key < len(self.value):
            raise IndexError("JsonValue: array index out of range")
        return JsonValue(self.value[key])

    def at_or_null(self, index: int) -> "JsonValue":
        return JsonValue(self.value[index] if isinstance(self.value, list) and 0 <= index < len(self.value) else None)

    def to_string(self) -> str: return self.dump()

    def dump(self) -> str:
        import json
        return json.dumps(self.value, separators=(",", ":"))

    @staticmethod
    def try_parse(text: str):
        """(value, error): a null node and the parser's message instead of an exception."""
        import json
        try:
            return JsonValue(json.loads(text)), ""
        except json.JSONDecodeError as e:
            return JsonValue(None), str(e)


def json_escape_string(s: str) -> str:
    """The JSON spelling of a string without its quotes."""
    import json
    return json.dumps(s)[1:-1]


class TensorView:
    """A strided window onto storage that someone else owns: every operation returns another view of the same memory and
    never copies (``reshape`` refuses a view that is not contiguous rather than copying silently).  A torch tensor already
    is such a view; this class pins the no-copy contract and keeps the reference's interface (include/quant/tensor_view.h)."""

    def __init__(self, data, shape=None, strides=None, offset: int = 0):
        import torch
        base = data.t if isinstance(data, TensorView) else data
        if shape is None:
            self.t = base
        else:
            shape = tuple(shape)
            if strides is None:
                strides, acc = [], 1
                for d in reversed(shape):
                    strides.insert(0, acc)
                    acc *= d
            self.t = torch.as_strided(base, shape, tuple(strides), base.storage_offset() + offset)

    def shape(self) -> Shape: return Shape(*self.t.shape)
    def strides(self): return list(self.t.stride())
    def rank(self) -> int: return self.t.dim()
    def numel(self) -> int: return self.t.numel()
    def dtype(self): return self.t.dtype
    def data(self): return self.t
    def data_ptr(self) -> int: return self.t.data_ptr()
    def is_contiguous(self) -> bool: return self.t.is_contiguous()

    def slice(self, dim: int, start: int, end: int) -> "TensorView":
        if not (0 <= dim < self.t.dim() and 0 <= start <= end <= self.t.shape[dim]):
            raise IndexError("TensorView.slice out of range")
        return TensorView(self.t.narrow(dim, start, end - start))

    def narrow(self, dim: int, start: int, size: int) -> "TensorView": return self.slice(dim, start, start + size)
    def transpose(self, d1: int, d2: int) -> "TensorView": return TensorView(self.t.transpose(d1, d2))
    def unsqueeze(self, dim: int) -> "TensorView": return TensorView(self.t.unsqueeze(dim))

    def squeeze(self, dim: int) -> "TensorView":
        if self.t.shape[dim] != 1:
            raise ValueError("TensorView.squeeze: the dimension is not 1")
        return TensorView(self.t.squeeze(dim))

    def reshape(self, *shape) -> "TensorView":
        if not self.t.is_contiguous():
            raise ValueError("only a contiguous view can be reshaped without a copy")
        return TensorView(self.t.view(*shape))

    def contiguous(self):
        """An owning, densely packed copy (a plain tensor)."""
        return self.t.contiguous().clone() if self.t.is_contiguous() else self.t.contiguous()

    def at(self, *index):
        return self.t[tuple(index)].item()
