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
    """Indexable collection of samples.  Pythonic access (``len``, ``[]``, iteration, ``map / filter / shuffle / concat``)
    and the reference's verbs ``size()`` / ``get(i)`` (include/quant/dataset.h:18-24) are the same thing."""

    def __len__(self):
        raise NotImplementedError

    def __getitem__(self, i):
        raise NotImplementedError

    def size(self) -> int:
        return len(self)

    def get(self, i):
        return self[i]

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


def _windows(tokens, seq_len: int, stride: int = -1, max_samples: int = -1):
    """(input, target) pairs of ``seq_len`` tokens, targets shifted by one, windows ``stride`` apart."""
    t = torch.as_tensor(tokens, dtype=torch.long).reshape(-1)
    stride = seq_len if stride is None or stride <= 0 else stride
    out = []
    for o in range(0, t.numel() - seq_len, stride):
        out.append((t[o:o + seq_len].clone(), t[o + 1:o + seq_len + 1].clone()))
        if 0 < max_samples <= len(out):
            break
    return out


class InMemoryDataset(Dataset):
    def __init__(self, items: Sequence = ()):
        self.items = list(items)

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]

    # ---- (input, target) samples: the reference's form (include/quant/dataset.h:26-49)
    def add_sample(self, inp, target):
        self.items.append((inp, target))

    def clear(self):
        self.items = []

    def inputs(self):
        return [it[0] for it in self.items]

    def targets(self):
        return [it[1] for it in self.items]

    @classmethod
    def from_text_file(cls, path, tok, seq_len: int, stride: int = -1, max_samples: int = -1) -> "InMemoryDataset":
        """Tokenise a text file and cut it into next-token windows."""
        text = open(path, "r", encoding="utf-8", errors="ignore").read()
        return cls(_windows(tok.encode(text), seq_len, stride, max_samples))

    @classmethod
    def from_tokenized_file(cls, path, seq_len: int, max_samples: int = -1, dtype=np.int64) -> "InMemoryDataset":
        """A flat binary file of token ids (int64 as the reference writes them; ``dtype`` for other widths)."""
        return cls(_windows(np.fromfile(path, dtype=dtype).astype(np.int64), seq_len, -1, max_samples))

    @classmethod
    def from_directory(cls, directory, ext: str, tok, seq_len: int) -> "InMemoryDataset":
        ds = cls()
        for name in sorted(os.listdir(directory)):
            if name.endswith(ext):
                ds.items += cls.from_text_file(os.path.join(directory, name), tok, seq_len).items
        return ds


class MapDataset(Dataset):
    def __init__(self, base, fn):
        self.base, self.fn = base, fn

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        it = self.base[i]
        try:
            return self.fn(it)
        except TypeError:
            if isinstance(it, tuple) and len(it) == 2:          # a function of (input, target), the reference's form
                return self.fn(*it)
            raise

    def set_map_fn(self, fn):
        self.fn = fn


class FilterDataset(Dataset):
    def __init__(self, base, pred):
        self.base, self.pred = base, pred
        self.apply_filter()

    def _keep(self, it):
        try:
            return self.pred(it)
        except TypeError:
            if isinstance(it, tuple) and len(it) == 2:
                return self.pred(*it)
            raise

    def apply_filter(self):
        """Evaluate the predicate over the base again (after the base or the predicate changed)."""
        self.idx = [i for i in range(len(self.base)) if self._keep(self.base[i])]

    def filtered_indices(self):
        return list(self.idx)

    def __len__(self):
        return len(self.idx)

    def __getitem__(self, i):
        return self.base[self.idx[i]]


class ConcatDataset(Dataset):
    def __init__(self, parts=()):
        self.parts = list(parts)
        self.offsets = np.cumsum([0] + [len(p) for p in self.parts])

    def add_dataset(self, ds):
        self.parts.append(ds)
        self.offsets = np.cumsum([0] + [len(p) for p in self.parts])

    def num_datasets(self) -> int:
        return len(self.parts)

    def __len__(self):
        return int(self.offsets[-1])

    def __getitem__(self, i):
        k = int(np.searchsorted(self.offsets, i, side="right")) - 1
        return self.parts[k][i - int(self.offsets[k])]


class ShuffleDataset(Dataset):
    def __init__(self, base, seed=42, buffer_size: int = 0):
        self.base, self._rng, self.buffer_size = base, Xoroshiro128Plus(seed), buffer_size
        self.reshuffle()

    def reshuffle(self):
        """A new permutation.  With ``buffer_size`` > 0 the shuffle is local: indices move only within consecutive
        windows of that many samples (what a bounded shuffle buffer over a stream achieves)."""
        n = len(self.base)
        if self.buffer_size and self.buffer_size < n:
            perm = []
            for o in range(0, n, self.buffer_size):
                perm += self._rng.shuffle(list(range(o, min(n, o + self.buffer_size))))
            self.perm = perm
        else:
            self.perm = self._rng.shuffle(list(range(n)))

    def permutation(self):
        return list(self.perm)

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        return self.base[self.perm[i]]


class ChunkedDataset(Dataset):
    """Fixed-length windows over one long token sequence."""

    def __init__(self, tokens, chunk: int, stride: Optional[int] = None, overlap: int = 0):
        """``tokens``: a sequence of ids, or the path of a flat int64 token file (mapped, not loaded)."""
        if isinstance(tokens, (str, os.PathLike)):
            tokens = np.memmap(tokens, dtype=np.int64, mode="r")
        self.t, self.c = tokens, chunk
        self.s = stride or max(1, chunk - overlap)

    def num_chunks(self) -> int:
        return len(self)

    def set_overlap(self, overlap: int):
        self.s = max(1, self.c - overlap)

    def __len__(self):
        return max(0, (len(self.t) - self.c) // self.s + 1)

    def __getitem__(self, i):
        o = i * self.s
        return self.t[o:o + self.c]


class StreamingDataset:
    """Iterates lines of (possibly many, possibly huge) text files without loading them.

    With ``seq_len`` the files are token shards (whitespace-separated integer ids, the reference's shard format,
    src/core/dataset.cpp:234-290) that are read through a bounded buffer: ``next_chunk(n)`` hands out the next n ids,
    ``get(i)`` the next (input, target) window, ``shuffle()`` reorders the shards, ``reset()`` starts over."""

    def __init__(self, paths, seq_len: Optional[int] = None, buffer_size: int = 10000, seed: int = 42):
        if isinstance(paths, (str, os.PathLike)):
            import glob
            paths = sorted(glob.glob(str(paths))) or [str(paths)]
        self.paths = list(paths)
        self.seq_len, self.buffer_size = seq_len, buffer_size
        self._rng = Xoroshiro128Plus(seed)
        self._order = list(range(len(self.paths)))
        self.reset()

    # ---- token-shard mode
    def reset(self):
        self._shard, self._fh, self._buf, self._carry, self._done = 0, None, [], "", False

    def shuffle(self):
        self._order = self._rng.shuffle(list(range(len(self.paths))))
        self.reset()

    def _refill(self, want: int):
        while len(self._buf) < want and not self._done:
            if self._fh is None:
                if self._shard >= len(self._order):
                    self._done = True
                    break
                self._fh = open(self.paths[self._order[self._shard]], "r")
            block = self._fh.read(max(4096, 8 * min(want, self.buffer_size)))
            if not block:
                self._fh.close()
                self._fh, self._shard = None, self._shard + 1
                if self._carry.strip():
                    self._buf.append(int(self._carry))
                self._carry = ""
                continue
            block = self._carry + block
            cut = max(block.rfind(" "), block.rfind("\n"), block.rfind("\t"))
            self._carry, block = (block[cut + 1:], block[:cut]) if cut >= 0 else (block, "")
            self._buf += [int(x) for x in block.split()]

    def has_next(self) -> bool:
        self._refill(1)
        return bool(self._buf)

    def next_chunk(self, chunk_size: int) -> List[int]:
        self._refill(chunk_size)
        out, self._buf = self._buf[:chunk_size], self._buf[chunk_size:]
        return out

    def get(self, index: int = 0):
        """The next (input, target) window of ``seq_len`` ids (the stream is sequential: ``index`` is not used)."""
        ids = self.next_chunk(self.seq_len + 1)
        if len(ids) < self.seq_len + 1:
            raise IndexError("the stream is exhausted")
        self._buf = ids[-1:] + self._buf                       # the last id starts the next window
        t = torch.tensor(ids, dtype=torch.long)
        return t[:-1], t[1:]

    def size(self) -> int:
        """Estimate of the number of ids in all shards (from the file sizes; about 4 characters per id)."""
        return sum(os.path.getsize(p) for p in self.paths) // 4

    def num_chunks(self) -> int:
        return self.size() // max(1, self.seq_len or 1)

    # ---- batch form (reference: StreamingDataset, include/quant/parquet_streamer.h:36-63)
    def add_shard(self, path: str):
        self.paths.append(str(path))
        self._order.append(len(self.paths) - 1)
        self._done = False

    def shuffle_shards(self): self.shuffle()
    def shards_loaded(self) -> int: return len(self.paths)
    def epochs_completed(self) -> int: return getattr(self, "_epochs", 0)
    def total_tokens(self) -> int: return getattr(self, "_served", 0)

    def next_batch(self, batch_size: int, seq_len: Optional[int] = None):
        """(input_ids, labels), both int64 [batch_size, seq_len], cut from the stream as consecutive windows of seq_len + 1
        ids.  When the shards run out before the batch is full the stream starts over (one more epoch completed) and the
        batch is filled from the start; None when the shards hold less than one window."""
        S = seq_len or self.seq_len
        rows: List[List[int]] = []
        wrapped = False
        while len(rows) < batch_size:
            ids = self.next_chunk(S + 1)
            if len(ids) < S + 1:
                if wrapped:
                    return None
                self._epochs = self.epochs_completed() + 1
                self.reset()
                wrapped = True
                continue
            rows.append(ids)
            wrapped = False
        t = torch.tensor(rows, dtype=torch.long)
        self._served = self.total_tokens() + batch_size * S
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()

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
    """Text clean-up before tokenisation: Unicode normalisation, control characters, whitespace, and the optional passes
    of the reference (HTML tags, URLs, e-mail addresses, personal identifiers, accents, length limits, exact and fuzzy
    de-duplication; include/quant/dataloader.h:29-86)."""

    _URL = re.compile(r"(?:https?://|www\.)\S+", re.I)
    _EMAIL = re.compile(r"[\w.+-]+@[\w-]+(?:\.[\w-]+)+")
    _TAG = re.compile(r"<(?:script|style)\b.*?</(?:script|style)>|<[^>]{1,200}>", re.I | re.S)
    _PII = (re.compile(r"\b\d{3}-\d{2}-\d{4}\b"),                                  # social-security-number shape
            re.compile(r"\b(?:\d[ -]?){13,16}\b"),                                 # payment-card shape
            re.compile(r"(?<!\w)(?:\+?\d{1,3}[ .-]?)?(?:\(\d{2,4}\)[ .-]?)?\d{3,4}[ .-]\d{3,4}(?:[ .-]\d{2,4})?(?!\w)"),
            re.compile(r"\b(?:\d{1,3}\.){3}\d{1,3}\b"))                            # IPv4 address

    def __init__(self, lowercase=False, normalize="NFKC", strip_control=True, collapse_whitespace=True, min_chars=0):
        self.lower, self.norm, self.ctrl, self.ws, self.min_chars = lowercase, normalize, strip_control, collapse_whitespace, min_chars
        self.accents = self.html = self.urls = self.emails = self.pii = self.dedup = False
        self.fuzzy_threshold, self.max_chars = 0.95, -1

    # ---- switches with the reference's names
    def set_lowercase(self, v): self.lower = bool(v)
    def set_accent_removal(self, v): self.accents = bool(v)
    def set_html_stripping(self, v): self.html = bool(v)
    def set_url_removal(self, v): self.urls = bool(v)
    def set_email_removal(self, v): self.emails = bool(v)
    def set_whitespace_normalization(self, v): self.ws = bool(v)
    def set_pii_removal(self, v): self.pii = bool(v)
    def set_deduplication(self, v): self.dedup = bool(v)
    def set_fuzzy_dedup_threshold(self, t): self.fuzzy_threshold = float(t)
    def set_min_length(self, n): self.min_chars = int(n)
    def set_max_length(self, n): self.max_chars = int(n)

    def __call__(self, s: str) -> str:
        if self.norm:
            s = unicodedata.normalize(self.norm, s)
        if self.html:
            s = self._TAG.sub(" ", s)
        if self.urls:
            s = self._URL.sub(" ", s)
        if self.emails:
            s = self._EMAIL.sub(" ", s)
        if self.pii:
            s = self._EMAIL.sub("[EMAIL]", s)
            for rx in self._PII:
                s = rx.sub("[REDACTED]", s)
        if self.accents:
            s = "".join(ch for ch in unicodedata.normalize("NFD", s) if unicodedata.category(ch) != "Mn")
        if self.ctrl:
            s = "".join(ch for ch in s if ch in "\n\t" or unicodedata.category(ch)[0] != "C")
        if self.ws:
            s = re.sub(r"[ \t]+", " ", s).strip()
        if self.max_chars >= 0:
            s = s[: self.max_chars]
        return s.lower() if self.lower else s

    def keep(self, s: str) -> bool:
        return len(s) >= self.min_chars

    def process(self, text: str) -> str:
        """Cleaned text, or "" when it falls under the minimum length."""
        out = self(text)
        return out if self.keep(out) else ""

    def process_batch(self, texts: Sequence[str]) -> List[str]:
        out = [t for t in (self.process(x) for x in texts) if t]
        return self.deduplicate(out) if self.dedup else out

    @staticmethod
    def fuzzy_similarity(a: str, b: str) -> float:
        """Jaccard similarity of the two texts' character trigrams."""
        ga = {a[i:i + 3] for i in range(max(1, len(a) - 2))}
        gb = {b[i:i + 3] for i in range(max(1, len(b) - 2))}
        return len(ga & gb) / max(1, len(ga | gb))

    def deduplicate(self, texts: Sequence[str]) -> List[str]:
        """Drop exact repeats, then texts whose trigram similarity to an earlier kept text reaches the threshold."""
        seen, kept = set(), []
        for t in texts:
            if t in seen:
                continue
            seen.add(t)
            if self.fuzzy_threshold < 1.0 and any(abs(len(t) - len(k)) <= 0.2 * max(len(t), len(k)) and
                                                  self.fuzzy_similarity(t, k) >= self.fuzzy_threshold for k in kept):
                continue
            kept.append(t)
        return kept

    @staticmethod
    def detect_language(text: str) -> str:
        """Coarse script / stop-word guess: "zh", "ja", "ko", "ru", "ar", "hi", a few Latin-script languages, else "unknown"."""
        counts = {}
        for ch in text:
            o = ord(ch)
            k = ("ja" if 0x3040 <= o <= 0x30FF else "zh" if 0x4E00 <= o <= 0x9FFF else "ko" if 0xAC00 <= o <= 0xD7AF else
                 "ru" if 0x0400 <= o <= 0x04FF else "ar" if 0x0600 <= o <= 0x06FF else "hi" if 0x0900 <= o <= 0x097F else
                 "latin" if ch.isalpha() and o < 0x250 else None)
            if k:
                counts[k] = counts.get(k, 0) + 1
        if not counts:
            return "unknown"
        if counts.get("ja", 0) > 0 and counts.get("ja", 0) + counts.get("zh", 0) >= max(counts.values()):
            return "ja"
        top = max(counts, key=counts.get)
        if top != "latin":
            return top
        words = set(re.findall(r"[a-zà-ÿ]+", text.lower()))
        stops = {"en": {"the", "and", "of", "to", "is", "in", "that"}, "es": {"el", "la", "de", "que", "y", "los", "es"},
                 "fr": {"le", "la", "les", "de", "et", "est", "des", "une"}, "de": {"der", "die", "und", "das", "ist", "nicht", "ein"},
                 "it": {"il", "di", "che", "è", "per", "una", "gli"}, "pt": {"o", "de", "que", "não", "uma", "os", "para"}}
        best = max(stops, key=lambda k: len(words & stops[k]))
        return best if words & stops[best] else "unknown"

    def process_with_metadata(self, texts: Sequence[str]):
        """(cleaned texts, language of each, length of each) for the texts that survive the clean-up."""
        out = self.process_batch(texts)
        return out, [self.detect_language(t) for t in out], [len(t) for t in out]


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

    next_batch_with_labels = next_batch

    def num_batches(self) -> int:
        return len(self)

    def has_next(self) -> bool:
        """Random windows never run out; the loader reports a next batch as long as one window fits."""
        return len(self.tokens) > self.S + 1

    def reset(self, seed: Optional[int] = None):
        if seed is not None:
            self.rng = Xoroshiro128Plus(seed)

    def dedup(self, window: int = 256, deduper: Optional["MinHashDeduper"] = None):
        """Near-duplicate report over consecutive ``window``-token spans (MinHash over token n-grams): returns the indices
        of the spans that repeat an earlier one.  The file is not modified."""
        d = deduper or MinHashDeduper(shingle=4, threshold=0.8)
        dups = []
        for i in range(len(self.tokens) // window):
            if d.is_duplicate(" ".join(map(str, self.tokens[i * window:(i + 1) * window].tolist()))):
                dups.append(i)
        return dups

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

    # ---- the reference's verbs (include/quant/trainer.h:160-238)
    def batch_size(self) -> int: return self.B
    def seq_length(self) -> int: return self.S

    def next_batch(self):
        """The next (ids, labels) pair, or None when the stream has ended."""
        if getattr(self, "_ended", False):
            return None
        item = self.q.get()
        if item is None:
            self._ended = True
            return None
        return item[0].to(self.device, non_blocking=True), item[1].to(self.device, non_blocking=True)

    def num_batches(self) -> int:
        """Estimate from the files' sizes (about one token per 4 bytes of text)."""
        import os
        return sum(os.path.getsize(p) for p in self.paths) // 4 // max(1, self.B * (self.S + 1))

    def reset(self):
        """Start the stream over: the worker is stopped and a new one reads the files from the beginning."""
        self.close()
        self.thread.join(timeout=5)
        self.q = queue.Queue(maxsize=self.q.maxsize)
        self._stop, self._ended = False, False
        self.thread = threading.Thread(target=self._work, daemon=True)
        self.thread.start()

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

    # ---- the reference's task generators (include/quant/data_gen.h:14-52): one text sample per entry
    _WORDS = ("the", "a", "model", "data", "learns", "reads", "fast", "small", "token", "layer", "writes", "tests", "code",
              "graph", "kernel", "memory", "sorts", "copies", "adds", "finds")

    def _word(self): return self._WORDS[self.rng.randint(0, len(self._WORDS))]
    def _letters(self, n): return "".join(chr(97 + self.rng.randint(0, 26)) for _ in range(n))

    def generate_random_text(self, num_samples, avg_length, vocab_size=100):
        vocab = [f"w{i}" for i in range(vocab_size)]
        return [" ".join(vocab[self.rng.randint(0, vocab_size)] for _ in range(max(1, avg_length // 2 + self.rng.randint(0, avg_length + 1))))
                for _ in range(num_samples)]

    def generate_arithmetic(self, num_samples, ops="+-"):
        out = []
        for _ in range(num_samples):
            a, b, op = self.rng.randint(0, 100), self.rng.randint(0, 100), ops[self.rng.randint(0, len(ops))]
            if op == "/":
                b = max(1, b)
                a = a - a % b
            val = {"+": a + b, "-": a - b, "*": a * b, "/": a // max(1, b)}[op]
            out.append(f"{a} {op} {b} = {val}")
        return out

    def generate_pattern_recognition(self, num_samples, pattern_length=4):
        out = []
        for _ in range(num_samples):
            pat = [str(self.rng.randint(0, 10)) for _ in range(pattern_length)]
            out.append(" ".join(pat * 3) + " -> " + " ".join(pat))
        return out

    def generate_copy_tasks(self, num_samples, max_length=50):
        return [f"copy: {s} -> {s}" for s in (self._letters(1 + self.rng.randint(0, max_length)) for _ in range(num_samples))]

    def generate_reverse_tasks(self, num_samples, max_length=30):
        return [f"reverse: {s} -> {s[::-1]}" for s in (self._letters(1 + self.rng.randint(0, max_length)) for _ in range(num_samples))]

    def generate_sorting_tasks(self, num_samples, max_items=10):
        out = []
        for _ in range(num_samples):
            xs = [self.rng.randint(0, 100) for _ in range(2 + self.rng.randint(0, max(1, max_items - 1)))]
            out.append("sort: " + " ".join(map(str, xs)) + " -> " + " ".join(map(str, sorted(xs))))
        return out

    def generate_ngram_text(self, num_samples, avg_length, ngram_order=3):
        """Text from a fixed random n-gram chain: the next word depends on the previous ``ngram_order - 1`` words."""
        out = []
        W = len(self._WORDS)
        for _ in range(num_samples):
            ctx = [self.rng.randint(0, W) for _ in range(max(1, ngram_order - 1))]
            words = [self._WORDS[i] for i in ctx]
            for _ in range(max(1, avg_length)):
                h = 1469598103934665603
                for c in ctx:
                    h = ((h ^ (c + 1)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
                nxt = (h >> 7) % W if self.rng.uniform() < 0.8 else self.rng.randint(0, W)
                words.append(self._WORDS[nxt])
                ctx = ctx[1:] + [nxt]
            out.append(" ".join(words))
        return out

    def generate_masked_prediction(self, num_samples, sentence_length=10):
        out = []
        for _ in range(num_samples):
            ws = [self._word() for _ in range(sentence_length)]
            i = self.rng.randint(0, sentence_length)
            out.append(" ".join(ws[:i] + ["[MASK]"] + ws[i + 1:]) + " -> " + ws[i])
        return out

    def generate_next_token_prediction(self, num_samples, seq_length=20):
        out = []
        for _ in range(num_samples):
            start, step = self.rng.randint(0, 50), 1 + self.rng.randint(0, 5)
            xs = [start + step * i for i in range(seq_length + 1)]
            out.append(" ".join(map(str, xs[:-1])) + " -> " + str(xs[-1]))
        return out

    def generate_token_recovery(self, num_samples, seq_length=15):
        out = []
        for _ in range(num_samples):
            ws = [self._word() for _ in range(seq_length)]
            noisy = [w if self.rng.uniform() > 0.2 else "_" * len(w) for w in ws]
            out.append(" ".join(noisy) + " -> " + " ".join(ws))
        return out

    def generate_mixed(self, num_samples, task_weights: Optional[Sequence[float]] = None):
        """Samples drawn from the ten generators above in proportion to ``task_weights`` (uniform when omitted)."""
        gens = [lambda: self.generate_random_text(1, 12), lambda: self.generate_arithmetic(1), lambda: self.generate_pattern_recognition(1),
                lambda: self.generate_copy_tasks(1, 12), lambda: self.generate_reverse_tasks(1, 12), lambda: self.generate_sorting_tasks(1, 6),
                lambda: self.generate_ngram_text(1, 12), lambda: self.generate_masked_prediction(1), lambda: self.generate_next_token_prediction(1, 8),
                lambda: self.generate_token_recovery(1, 8)]
        w = list(task_weights or [1.0] * len(gens))[: len(gens)]
        w += [0.0] * (len(gens) - len(w))
        cdf = np.cumsum(np.asarray(w, dtype=np.float64) / max(1e-12, float(sum(w))))
        return [gens[min(len(gens) - 1, int(np.searchsorted(cdf, self.rng.uniform())))]()[0] for _ in range(num_samples)]

    def templated(self, n, templates: Sequence[str], slots: dict):
        out = []
        for _ in range(n):
            t = templates[self.rng.randint(0, len(templates))]
            out.append(re.sub(r"\{(\w+)\}", lambda m: slots[m.group(1)][self.rng.randint(0, len(slots[m.group(1)]))], t))
        return out


class CurriculumGenerator:
    """Orders samples from easy to hard and reveals them progressively: at progress p in [0, 1] the pool is the easiest
    ``start + (1 - start) * p`` fraction."""

    def __init__(self, samples: Sequence = (), difficulty: Optional[Callable] = None, start_fraction=0.2, seed=42):
        self.sorted = sorted(samples, key=difficulty) if difficulty is not None else list(samples)
        self.start, self.rng = start_fraction, Xoroshiro128Plus(seed)
        self.stages: List[dict] = []
        self._stage = self._stage_samples = self._acc_n = 0
        self._acc = 0.0
        self._progress_fn = None

    # ---- staged form (reference: include/quant/data_gen.h:54-80): generators ordered by difficulty; the learner's
    # reported accuracy promotes it to the next stage
    def add_stage(self, name: str, difficulty: int, generator_fn: Callable[[int], List[str]], max_samples: int = 10000,
                  accuracy_threshold: float = 0.9):
        self.stages.append(dict(name=name, difficulty=difficulty, fn=generator_fn, max_samples=max_samples, thr=accuracy_threshold))
        self.stages.sort(key=lambda st: st["difficulty"])

    def set_progress_fn(self, fn: Callable[[str, int, float], None]):
        self._progress_fn = fn

    def current_stage_name(self) -> str:
        return self.stages[self._stage]["name"] if self.stages and not self.is_complete() else ""

    def current_difficulty(self) -> int:
        return self.stages[min(self._stage, len(self.stages) - 1)]["difficulty"] if self.stages else 0

    def is_complete(self) -> bool:
        return bool(self.stages) and self._stage >= len(self.stages)

    def generate_next_batch(self, batch_size: int) -> List[str]:
        if not self.stages or self.is_complete():
            return []
        st = self.stages[self._stage]
        out = list(st["fn"](batch_size))
        self._stage_samples += len(out)
        if self._stage_samples >= st["max_samples"]:
            self._promote()
        return out

    def report_accuracy(self, accuracy: float):
        """Running mean of the reported accuracies within the stage; reaching the stage's threshold promotes."""
        if not self.stages or self.is_complete():
            return
        self._acc_n += 1
        self._acc += (accuracy - self._acc) / self._acc_n
        if self._progress_fn:
            self._progress_fn(self.current_stage_name(), self.current_difficulty(), self._acc)
        if self._acc >= self.stages[self._stage]["thr"]:
            self._promote()

    def _promote(self):
        self._stage += 1
        self._stage_samples, self._acc, self._acc_n = 0, 0.0, 0

    def pool(self, progress: float):
        f = min(1.0, self.start + (1 - self.start) * max(0.0, progress))
        return self.sorted[: max(1, int(round(f * len(self.sorted))))]

    def sample(self, progress, k):
        p = self.pool(progress)
        return [p[self.rng.randint(0, len(p))] for _ in range(k)]


class ParquetReader:
    """Text column of Parquet files, row group by row group (needs pyarrow)."""

    def __init__(self, path=None, column="text"):
        self.pf, self.column = None, column
        self._rows = self._tokens = 0
        self._it = None
        if path is not None:
            self.open(path)

    def open(self, path) -> bool:
        import pyarrow.parquet as pq
        try:
            self.pf = pq.ParquetFile(path)
        except Exception:
            self.pf = None
            return False
        self.reset()
        return True

    def reset(self):
        self._rows = self._tokens = 0
        self._it = None

    def close(self):
        self.pf, self._it = None, None

    def rows_read(self) -> int: return self._rows
    def total_tokens(self) -> int: return self._tokens

    def next_batch(self, max_tokens: int, tokenizer=None) -> List[int]:
        """Token ids of the next rows, at most ``max_tokens`` of them (bytes of the text when no tokenizer is given); an
        empty list at the end of the file."""
        if self.pf is None:
            return []
        if self._it is None:
            self._it, self._left = iter(self), []
        out = self._left
        while len(out) < max_tokens:
            row = next(self._it, None)
            if row is None:
                break
            self._rows += 1
            out = out + (tokenizer.encode(row) if tokenizer is not None else list(row.encode("utf-8")))
        out, self._left = out[:max_tokens], out[max_tokens:]
        self._tokens += len(out)
        return out

    def num_rows(self):
        return self.pf.metadata.num_rows

    def __iter__(self):
        for g in range(self.pf.num_row_groups):
            for v in self.pf.read_row_group(g, columns=[self.column]).column(0).to_pylist():
                if v is not None:
                    yield v


class ParquetStreamingDataset(StreamingDataset):
    """The same batch interface over Parquet shards: the text column of every shard is tokenised on the fly (UTF-8 bytes
    folded into the vocabulary when no tokenizer is given) and served as (input, label) windows.  ``data_dir`` may be a
    directory (every ``*.parquet`` in it, sorted), a glob or empty (shards are then added one by one).
    Reference counterpart: StreamingDataset (include/quant/parquet_streamer.h:36-63)."""

    def __init__(self, data_dir: str = "", vocab_size: int = 256, tokenizer=None, column: str = "text", seq_len: Optional[int] = None, seed: int = 42):
        import glob
        paths: List[str] = []
        if data_dir:
            paths = sorted(glob.glob(os.path.join(data_dir, "*.parquet"))) if os.path.isdir(data_dir) else sorted(glob.glob(data_dir))
        self.vocab_size, self.tokenizer, self.column = vocab_size, tokenizer, column
        super().__init__(paths, seq_len=seq_len, seed=seed)

    def add_shard(self, path: str):
        if not ParquetReader().open(path):
            raise ValueError(f"not a Parquet file: {path}")
        super().add_shard(path)

    def reset(self):
        super().reset()
        self._reader = None

    def _refill(self, want: int):
        while len(self._buf) < want and not self._done:
            if self._reader is None:
                if self._shard >= len(self._order):
                    self._done = True
                    break
                self._reader = ParquetReader(self.paths[self._order[self._shard]], self.column)
            ids = self._reader.next_batch(max(want - len(self._buf), 4096), self.tokenizer)
            if not ids:
                self._reader, self._shard = None, self._shard + 1
                continue
            self._buf += ids if self.tokenizer is not None else [i % self.vocab_size for i in ids]

    def size(self) -> int:
        return sum(ParquetReader(p, self.column).num_rows() for p in self.paths)


class DataPipeline:
    """source -> clean -> filter -> dedup -> tokenise -> pack into fixed-length rows."""

    def __init__(self, tokenizer=None, seq_length: int = 2048, preprocessor: Optional[TextPreprocessor] = None,
                 dedup: Optional[MinHashDeduper] = None, filters: Sequence[Callable[[str], bool]] = ()):
        self.tok, self.S, self.pre, self.dedup, self.filters = tokenizer, seq_length, preprocessor or TextPreprocessor(), dedup, list(filters)
        self.stats = {"seen": 0, "filtered": 0, "duplicates": 0, "tokens": 0}
        self.batch_size, self.num_workers = 32, 1
        self.custom_stages: List = []
        self._processed = 0

    # ---- the reference's three-stage form (include/quant/dataloader.h:88-117)
    def set_preprocessor(self, p: TextPreprocessor): self.pre = p
    def set_tokenizer(self, t): self.tok = t
    def set_batch_size(self, n: int): self.batch_size = int(n)
    def set_seq_length(self, n: int): self.S = int(n)
    def set_num_workers(self, n: int): self.num_workers = max(1, int(n))
    def total_processed(self) -> int: return self._processed

    def add_stage(self, name: str, fn: Callable):
        """A custom stage: ``fn(texts) -> texts`` applied, in the order added, between clean-up and tokenisation."""
        self.custom_stages.append((name, fn))

    def clear_pipeline(self):
        self.custom_stages = []

    def run_stage1(self, raw_texts: Sequence[str]) -> List[str]:
        """Clean-up, length filter, optional de-duplication."""
        out = self.pre.process_batch(raw_texts)
        if self.dedup is not None:
            out = [t for t in out if not self.dedup.is_duplicate(t)]
        return out

    def run_stage2(self, texts: Sequence[str]) -> List[List[int]]:
        """Tokenisation (on ``num_workers`` threads when more than one)."""
        if self.num_workers > 1 and len(texts) > 1:
            from concurrent.futures import ThreadPoolExecutor
            with ThreadPoolExecutor(self.num_workers) as ex:
                return list(ex.map(self.tok.encode, texts))
        return [self.tok.encode(t) for t in texts]

    def run_stage3(self, tokenized: Sequence[Sequence[int]]) -> List[torch.Tensor]:
        """Pack all ids into rows of ``seq_length`` and group the rows into [batch, seq_length] tensors."""
        flat = [i for ids in tokenized for i in ids]
        n = len(flat) // self.S
        rows = torch.tensor(flat[: n * self.S], dtype=torch.long).view(n, self.S)
        return [rows[o:o + self.batch_size] for o in range(0, n, self.batch_size)]

    def process_texts(self, texts: Sequence[str]) -> List[torch.Tensor]:
        texts = self.run_stage1(texts)
        for _, fn in self.custom_stages:
            texts = fn(texts)
        self._processed += len(texts)
        return self.run_stage3(self.run_stage2(texts))

    def process_file(self, path) -> List[torch.Tensor]:
        return self.process_texts([ln.rstrip("\n") for ln in open(path, "r", encoding="utf-8", errors="ignore") if ln.strip()])

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


class TokenizerEvaluator:
    """Quality figures of a tokenizer on a text: compression, round-trip fidelity, coverage and vocabulary use
    (reference: TokenizerEvaluator, include/quant/data_gen.h:82-120)."""

    def __init__(self, tokenizer):
        self.tok = tokenizer

    def compression_ratio(self, text: str) -> float:
        """UTF-8 bytes per token."""
        return len(text.encode("utf-8")) / max(1, len(self.tok.encode(text)))

    def character_error_rate(self, original: str, reconstructed: str) -> float:
        """Levenshtein distance divided by the length of the original."""
        a, b = original, reconstructed
        prev = list(range(len(b) + 1))
        for i, ca in enumerate(a, 1):
            cur = [i]
            for j, cb in enumerate(b, 1):
                cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
            prev = cur
        return prev[-1] / max(1, len(a))

    def reconstruction_fidelity(self, text: str) -> float:
        return 1.0 - min(1.0, self.character_error_rate(text, self.tok.decode(self.tok.encode(text))))

    def re_encoding_accuracy(self, text: str) -> float:
        """Fraction of positions at which encode(decode(encode(text))) equals encode(text)."""
        a = self.tok.encode(text)
        b = self.tok.encode(self.tok.decode(a))
        return sum(x == y for x, y in zip(a, b)) / max(1, max(len(a), len(b)))

    def _unk(self):
        return getattr(self.tok, "unk_id", -1)

    def vocabulary_coverage(self, corpus: str) -> float:
        """Fraction of tokens that are not the unknown token."""
        ids = self.tok.encode(corpus)
        return sum(i != self._unk() for i in ids) / max(1, len(ids))

    def average_token_length(self, corpus: str) -> float:
        return len(corpus) / max(1, len(self.tok.encode(corpus)))

    def vocabulary_utilization(self, corpus: str) -> float:
        v = getattr(self.tok, "vocab_size", None)
        v = v() if callable(v) else v
        return len(set(self.tok.encode(corpus))) / max(1, int(v or 1))

    def byte_efficiency(self, text: str) -> float:
        """Bits of token ids (at the vocabulary's width) per bit of UTF-8 text: below 1 means the ids are smaller."""
        v = getattr(self.tok, "vocab_size", None)
        v = int((v() if callable(v) else v) or 256)
        bits = max(1, (v - 1).bit_length())
        return len(self.tok.encode(text)) * bits / max(1, 8 * len(text.encode("utf-8")))

    @staticmethod
    def report_string(report: dict) -> str:
        """One aligned ``name: value`` line per figure of an ``evaluate`` result."""
        w = max((len(k) for k in report), default=0)
        return "\n".join(f"{k:<{w}} : {v:.4f}" if isinstance(v, float) else f"{k:<{w}} : {v}" for k, v in report.items())

    @staticmethod
    def compare_tokenizers(tokenizers, corpus) -> List[dict]:
        """The ``evaluate`` report of every tokenizer on the same corpus (a string, or documents that are joined by newlines),
        each with the tokenizer's class name under ``"tokenizer"``."""
        text = corpus if isinstance(corpus, str) else "\n".join(corpus)
        out = []
        for t in tokenizers:
            r = TokenizerEvaluator(t).evaluate(text)
            r["tokenizer"] = type(t).__name__
            out.append(r)
        return out

    def evaluate(self, corpus: str) -> dict:
        if not isinstance(corpus, str):
            corpus = "\n".join(corpus)
        ids = self.tok.encode(corpus)
        back = self.tok.decode(ids)
        return {"compression_ratio": self.compression_ratio(corpus), "re_encoding_accuracy": self.re_encoding_accuracy(corpus),
                "vocabulary_coverage": self.vocabulary_coverage(corpus), "average_token_length": self.average_token_length(corpus),
                "vocabulary_utilization": self.vocabulary_utilization(corpus), "reconstruction_fidelity": self.reconstruction_fidelity(corpus),
                "byte_efficiency": self.byte_efficiency(corpus), "character_error_rate": self.character_error_rate(corpus, back),
                "total_tokens": len(ids), "unique_tokens": len(set(ids)), "oov_count": sum(i == self._unk() for i in ids),
                "corpus_size_bytes": len(corpus.encode("utf-8"))}
