"""Datasets and data pipelines: composable dataset views, splitting, synthetic and curriculum generators, a memory-mapped
token loader with MinHash near-duplicate removal, text clean-up, a streaming loader with a prefetch thread and a Parquet
column reader.  Reference counterparts: include/quant/dataset.h:18-204, data_gen.h:14-91, mmap_dataloader.h:47-110,
dataloader.h:18-121, parquet_streamer.h:9-36, StreamingDataLoader (include/quant/trainer.h:160-238)."""
from __future__ import annotations

import hashlib
import mmap
import os
import queue
import re
import threading
import unicodedata
from typing import Callable, Iterable, Iterator, List, Optional, Sequence

import numpy as np
import torch

from .random import Xoroshiro128Plus


class Dataset:
    def __len__(self):
        raise NotImplementedError

    def __getitem__(self, i):
        raise NotImplementedError

    def __iter__(self):
        return (self[i] for i in range(len(self)))

    def map(self, fn):
        return MapDataset(self, fn)

    def filter(self, pred):
        return FilterDataset(self, pred)

    def shuffle(self, seed=42):
        return ShuffleDataset(self, seed)

    def concat(self, other):
        return ConcatDataset([self, other])


class InMemoryDataset(Dataset):
    def __init__(self, items: Sequence):
        self.items = list(items)

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]


class MapDataset(Dataset):
    def __init__(self, base, fn):
        self.base, self.fn = base, fn

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        return self.fn(self.base[i])


class FilterDataset(Dataset):
    def __init__(self, base, pred):
        self.base = base
        self.idx = [i for i in range(len(base)) if pred(base[i])]

    def __len__(self):
        return len(self.idx)

    def __getitem__(self, i):
        return self.base[self.idx[i]]


class ConcatDataset(Dataset):
    def __init__(self, parts):
        self.parts = list(parts)
        self.offsets = np.cumsum([0] + [len(p) for p in self.parts])

    def __len__(self):
        return int(self.offsets[-1])

    def __getitem__(self, i):
        k = int(np.searchsorted(self.offsets, i, side="right")) - 1
        return self.parts[k][i - int(self.offsets[k])]


class ShuffleDataset(Dataset):
    def __init__(self, base, seed=42):
        self.base = base
        self.perm = Xoroshiro128Plus(seed).shuffle(list(range(len(base))))

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        return self.base[self.perm[i]]


class ChunkedDataset(Dataset):
    """Fixed-length windows over one long token sequence."""

    def __init__(self, tokens: Sequence[int], chunk: int, stride: Optional[int] = None):
        self.t, self.c, self.s = tokens, chunk, stride or chunk

    def __len__(self):
        return max(0, (len(self.t) - self.c) // self.s + 1)

    def __getitem__(self, i):
        o = i * self.s
        return self.t[o:o + self.c]


class StreamingDataset:
    """Iterates lines of (possibly many, possibly huge) text files without loading them."""

    def __init__(self, paths: Sequence[str]):
        self.paths = list(paths)

    def __iter__(self) -> Iterator[str]:
        for p in self.paths:
            with open(p, "r", encoding="utf-8", errors="ignore") as f:
                for line in f:
                    yield line.rstrip("\n")


def split_dataset(ds: Dataset, fractions=(0.9, 0.05, 0.05), seed=42):
    perm = Xoroshiro128Plus(seed).shuffle(list(range(len(ds))))
    out, o = [], 0
    for k, f in enumerate(fractions):
        n = len(ds) - o if k == len(fractions) - 1 else int(round(f * len(ds)))
        idx = perm[o:o + n]
        out.append(InMemoryDataset([ds[i] for i in idx]))
        o += n
    return out


class TextPreprocessor:
    def __init__(self, lowercase=False, normalize="NFKC", strip_control=True, collapse_whitespace=True, min_chars=0):
        self.lower, self.norm, self.ctrl, self.ws, self.min_chars = lowercase, normalize, strip_control, collapse_whitespace, min_chars

    def __call__(self, s: str) -> str:
        if self.norm:
            s = unicodedata.normalize(self.norm, s)
        if self.ctrl:
            s = "".join(ch for ch in s if ch in "\n\t" or unicodedata.category(ch)[0] != "C")
        if self.ws:
            s = re.sub(r"[ \t]+", " ", s).strip()
        return s.lower() if self.lower else s

    def keep(self, s: str) -> bool:
        return len(s) >= self.min_chars


class MinHashDeduper:
    """Near-duplicate filter: ``num_perm`` min-hashes over word ``shingle``-grams, banded LSH; a document is dropped when a
    band matches an earlier document and the estimated Jaccard similarity reaches ``threshold``."""

    def __init__(self, num_perm=64, bands=16, shingle=3, threshold=0.8, seed=1):
        rng = Xoroshiro128Plus(seed)
        self.a = np.array([rng.next_u64() | 1 for _ in range(num_perm)], dtype=np.uint64)
        self.b = np.array([rng.next_u64() for _ in range(num_perm)], dtype=np.uint64)
        self.bands, self.rows, self.k, self.thr = bands, num_perm // bands, shingle, threshold
        self.buckets = [dict() for _ in range(bands)]
        self.sigs: List[np.ndarray] = []

    def signature(self, text: str) -> np.ndarray:
        w = text.split()
        grams = {" ".join(w[i:i + self.k]) for i in range(max(1, len(w) - self.k + 1))}
        h = np.array([int.from_bytes(hashlib.blake2b(g.encode(), digest_size=8).digest(), "little") for g in grams], dtype=np.uint64)
        with np.errstate(over="ignore"):
            return (self.a[:, None] * h[None, :] + self.b[:, None]).min(1)

    def is_duplicate(self, text: str, add=True) -> bool:
        sig = self.signature(text)
        cands = set()
        keys = [sig[i * self.rows:(i + 1) * self.rows].tobytes() for i in range(self.bands)]
        for i, k in enumerate(keys):
            cands.update(self.buckets[i].get(k, ()))
        dup = any(float((self.sigs[c] == sig).mean()) >= self.thr for c in cands)
        if add and not dup:
            idx = len(self.sigs)
            self.sigs.append(sig)
            for i, k in enumerate(keys):
                self.buckets[i].setdefault(k, []).append(idx)
        return dup


class MmapDataLoader:
    """Token ids in a flat binary file (uint16 or int32) mapped into memory; batches are random windows."""

    def __init__(self, path, batch_size, seq_length, dtype=np.uint16, seed=42):
        self.f = open(path, "rb")
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ)
        self.tokens = np.frombuffer(self.mm, dtype=dtype)
        self.B, self.S = batch_size, seq_length
        self.rng = Xoroshiro128Plus(seed)

    def __len__(self):
        return max(0, (len(self.tokens) - 1) // (self.B * self.S))

    def next_batch(self):
        hi = len(self.tokens) - self.S - 1
        starts = [self.rng.randint(0, max(1, hi)) for _ in range(self.B)]
        x = np.stack([self.tokens[s:s + self.S + 1] for s in starts]).astype(np.int64)
        t = torch.from_numpy(x)
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()

    @staticmethod
    def write_tokens(path, tokens, dtype=np.uint16):
        np.asarray(tokens, dtype=dtype).tofile(path)

    def close(self):
        self.tokens = None
        self.mm.close()
        self.f.close()


class StreamingDataLoader:
    """Tokenises text files on a background thread and hands out [B, S] batches through a bounded queue."""

    def __init__(self, tokenizer, paths: Sequence[str], batch_size, seq_length, prefetch=4, device="cpu", loop=False):
        self.tok, self.paths, self.B, self.S, self.device, self.loop = tokenizer, list(paths), batch_size, seq_length, device, loop
        self.q: "queue.Queue" = queue.Queue(maxsize=prefetch)
        self._stop = False
        self.thread = threading.Thread(target=self._work, daemon=True)
        self.thread.start()

    def _work(self):
        need = self.B * (self.S + 1)
        buf: List[int] = []
        while not self._stop:
            for line in StreamingDataset(self.paths):
                if self._stop:
                    return
                buf += self.tok.encode(line + "\n")
                while len(buf) >= need:
                    chunk, buf = buf[:need], buf[need:]
                    t = torch.tensor(chunk, dtype=torch.long).view(self.B, self.S + 1)
                    self.q.put((t[:, :-1].contiguous(), t[:, 1:].contiguous()))
            if not self.loop:
                break
        self.q.put(None)

    def __iter__(self):
        while True:
            item = self.q.get()
            if item is None:
                return
            yield item[0].to(self.device, non_blocking=True), item[1].to(self.device, non_blocking=True)

    def close(self):
        self._stop = True
        while not self.q.empty():
            self.q.get_nowait()


class DataGenerator:
    """Synthetic corpora for tests and smoke runs: arithmetic, copy / reverse tasks, Zipfian token streams, templated text."""

    def __init__(self, seed=42):
        self.rng = Xoroshiro128Plus(seed)

    def arithmetic(self, n, max_value=99):
        out = []
        for _ in range(n):
            a, b = self.rng.randint(0, max_value + 1), self.rng.randint(0, max_value + 1)
            op = "+-*"[self.rng.randint(0, 3)]
            out.append(f"{a} {op} {b} = {eval(f'{a}{op}{b}')}")
        return out

    def copy_task(self, n, length=8, vocab=26, reverse=False):
        out = []
        for _ in range(n):
            s = "".join(chr(97 + self.rng.randint(0, vocab)) for _ in range(length))
            out.append(f"{s} -> {s[::-1] if reverse else s}")
        return out

    def zipf_tokens(self, n, vocab_size, exponent=1.1):
        w = 1.0 / np.arange(1, vocab_size + 1) ** exponent
        cdf = np.cumsum(w / w.sum())
        u = np.array([self.rng.uniform() for _ in range(n)])
        return np.minimum(np.searchsorted(cdf, u), vocab_size - 1).astype(np.int64)

    def templated(self, n, templates: Sequence[str], slots: dict):
        out = []
        for _ in range(n):
            t = templates[self.rng.randint(0, len(templates))]
            out.append(re.sub(r"\{(\w+)\}", lambda m: slots[m.group(1)][self.rng.randint(0, len(slots[m.group(1)]))], t))
        return out


class CurriculumGenerator:
    """Orders samples from easy to hard and reveals them progressively: at progress p in [0, 1] the pool is the easiest
    ``start + (1 - start) * p`` fraction."""

    def __init__(self, samples: Sequence, difficulty: Callable, start_fraction=0.2, seed=42):
        self.sorted = sorted(samples, key=difficulty)
        self.start, self.rng = start_fraction, Xoroshiro128Plus(seed)

    def pool(self, progress: float):
        f = min(1.0, self.start + (1 - self.start) * max(0.0, progress))
        return self.sorted[: max(1, int(round(f * len(self.sorted))))]

    def sample(self, progress, k):
        p = self.pool(progress)
        return [p[self.rng.randint(0, len(p))] for _ in range(k)]


class ParquetReader:
    """Text column of Parquet files, row group by row group (needs pyarrow)."""

    def __init__(self, path, column="text"):
        import pyarrow.parquet as pq
        self.pf, self.column = pq.ParquetFile(path), column

    def num_rows(self):
        return self.pf.metadata.num_rows

    def __iter__(self):
        for g in range(self.pf.num_row_groups):
            for v in self.pf.read_row_group(g, columns=[self.column]).column(0).to_pylist():
                if v is not None:
                    yield v


class DataPipeline:
    """source -> clean -> filter -> dedup -> tokenise -> pack into fixed-length rows."""

    def __init__(self, tokenizer, seq_length, preprocessor: Optional[TextPreprocessor] = None, dedup: Optional[MinHashDeduper] = None,
                 filters: Sequence[Callable[[str], bool]] = ()):
        self.tok, self.S, self.pre, self.dedup, self.filters = tokenizer, seq_length, preprocessor or TextPreprocessor(), dedup, list(filters)
        self.stats = {"seen": 0, "filtered": 0, "duplicates": 0, "tokens": 0}

    def run(self, docs: Iterable[str]) -> torch.Tensor:
        buf: List[int] = []
        for d in docs:
            self.stats["seen"] += 1
            d = self.pre(d)
            if not self.pre.keep(d) or not all(f(d) for f in self.filters):
                self.stats["filtered"] += 1
                continue
            if self.dedup is not None and self.dedup.is_duplicate(d):
                self.stats["duplicates"] += 1
                continue
            ids = self.tok.encode(d, add_eos=True) if "add_eos" in self.tok.encode.__code__.co_varnames else self.tok.encode(d)
            buf += ids
        self.stats["tokens"] = len(buf)
        n = len(buf) // self.S
        return torch.tensor(buf[: n * self.S], dtype=torch.long).view(n, self.S)
