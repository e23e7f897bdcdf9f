"""Deterministic random streams: splitmix64 seeding, xoroshiro128+ generator, Box-Muller normals, named seed streams and
seed resolution (command line > QUANT_SEED > 42).  Reference counterparts: include/quant/random.h, src/core/random.cpp:16,41,113."""
from __future__ import annotations

import math
import os
import threading

M64 = 0xFFFFFFFFFFFFFFFF


def splitmix64(x: int):
    """(next state, output)."""
    x = (x + 0x9E3779B97F4A7C15) & M64
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return x, z ^ (z >> 31)


class Xoroshiro128Plus:
    def __init__(self, seed: int = 42):
        st, self.s0 = splitmix64(seed & M64)
        _, self.s1 = splitmix64(st)
        self._spare = None

    @staticmethod
    def _rotl(x, k):
        return ((x << k) | (x >> (64 - k))) & M64

    def next_u64(self) -> int:
        s0, s1 = self.s0, self.s1
        r = (s0 + s1) & M64
        s1 ^= s0
        self.s0 = self._rotl(s0, 24) ^ s1 ^ ((s1 << 16) & M64)
        self.s1 = self._rotl(s1, 37)
        return r

    def uniform(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))

    def randint(self, lo, hi) -> int:
        return lo + self.next_u64() % (hi - lo)

    def normal(self, mean=0.0, std=1.0) -> float:
        if self._spare is not None:
            z, self._spare = self._spare, None
        else:
            u1, u2 = max(self.uniform(), 1e-300), self.uniform()
            r = math.sqrt(-2.0 * math.log(u1))
            z, self._spare = r * math.cos(2 * math.pi * u2), r * math.sin(2 * math.pi * u2)
        return mean + std * z

    def shuffle(self, xs):
        for i in range(len(xs) - 1, 0, -1):
            j = self.next_u64() % (i + 1)
            xs[i], xs[j] = xs[j], xs[i]
        return xs


class SeedStream:
    INIT, DATA, DROPOUT, SAMPLING, NOISE, AUGMENT = range(6)


def make_seed(base: int, stream: int, counter: int = 0) -> int:
    _, a = splitmix64((base ^ (stream * 0xD1B54A32D192ED03)) & M64)
    _, b = splitmix64((a + counter) & M64)
    return b


def resolve_base_seed(cli_seed: int = 0) -> int:
    if cli_seed:
        return int(cli_seed)
    try:
        return int(os.environ.get("QUANT_SEED", "") or 42)
    except ValueError:
        return 42


class GlobalSeedManager:
    """Process-wide base seed: the ``QUANT_SEED`` environment variable when it is set to a non-zero number (runs are then
    reproducible), otherwise 64 bits of operating-system entropy drawn once.  ``next_seed`` hands every caller (thread,
    worker, generator) its own offset from the base.  Reference counterpart: GlobalSeedManager (include/quant/random.h:16-25,
    src/core/random.cpp:13-44)."""
    _base = 0
    _counter = 0
    _lock = threading.Lock()

    @classmethod
    def get_seed(cls) -> int:
        with cls._lock:
            if cls._base == 0:
                env = os.environ.get("QUANT_SEED", "")
                try:
                    v = int(env) if env else 0
                except ValueError:
                    v = 0
                if not env:
                    v = int.from_bytes(os.urandom(8), "little")
                cls._base = (v & 0xFFFFFFFFFFFFFFFF) or 1
            return cls._base

    @classmethod
    def next_seed(cls) -> int:
        base = cls.get_seed()
        with cls._lock:
            cls._counter += 1
            return (base + cls._counter) & 0xFFFFFFFFFFFFFFFF

    @staticmethod
    def is_deterministic() -> bool:
        env = os.environ.get("QUANT_SEED", "")
        try:
            return bool(env) and int(env) != 0
        except ValueError:
            return False

    @classmethod
    def reset(cls):
        """Forget the cached base seed and the counter (the next ``get_seed`` reads the environment again)."""
        with cls._lock:
            cls._base = cls._counter = 0
