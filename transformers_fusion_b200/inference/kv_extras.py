"""KV-cache tiers beyond the device page pool, and the reference's small inference API classes.

* ``TieredKVStore``      - host / disk spill tier under the device pages: least-recently-used pages are written to a
  memory-mapped file by a background worker and brought back (``ensure_resident`` with a timeout) before they are
  attended over; multi-level page tables (12 index bits per level) address 4096^2 pages with two levels and
  4096^3 pages with three (the reference's "4M" and "1T" caches).
* ``CompressedKVCache``  - ternary keys / values (2 bits + one scale per 32 elements).
* ``flash_decoding``     - split-KV single-query attention on plain tensors (oracle of the paged decode kernel).
* ``ReasoningBudget``    - token caps for "thinking" phases (256 / 2048 / 8192).
* ``PagedAttention`` / ``ContinuousBatching`` - facades with the reference's method names over the engine.

Reference counterparts: PagedKVCacheBase / 4M / 1T (src/model/kv_cache.cpp:389-1271), CompressedKVCache, PrefixCache,
flash_decoding (src/inference/inference_kv.cpp:20-205), ReasoningBudget (include/quant/sampler.h), PagedAttention /
ContinuousBatching (include/quant/inference_opt.h:17-90)."""
from __future__ import annotations

import mmap
import os
import queue
import tempfile
import threading
import time
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

PAGE = 16


class PageTable:
    """Sparse multi-level table: logical page number -> physical page id.  ``levels`` x 12 bits of index."""

    FANOUT = 4096

    def __init__(self, levels=2):
        self.levels = levels
        self.root: Dict = {}
        self.count = 0

    def capacity_tokens(self):
        return (self.FANOUT ** self.levels) * PAGE

    def _path(self, lpn):
        return [(lpn >> (12 * (self.levels - 1 - i))) & (self.FANOUT - 1) for i in range(self.levels)]

    def set(self, lpn, phys):
        if lpn >= self.FANOUT ** self.levels:
            raise IndexError("logical page beyond the table's reach")
        node = self.root
        path = self._path(lpn)
        for k in path[:-1]:
            node = node.setdefault(k, {})
        if path[-1] not in node:
            self.count += 1
        node[path[-1]] = phys

    def get(self, lpn, default=None):
        node = self.root
        for k in self._path(lpn):
            if not isinstance(node, dict) or k not in node:
                return default
            node = node[k]
        return node

    def pop(self, lpn):
        node, path = self.root, self._path(lpn)
        for k in path[:-1]:
            node = node.get(k, {})
        if path[-1] in node:
            self.count -= 1
            return node.pop(path[-1])
        return None


class TieredKVStore:
    """``resident_pages`` page slots in a fast tensor (device or pinned host) backed by a disk file holding every page.
    Page payload: [2 (k, v), PAGE, heads, dim] in ``dtype``."""

    def __init__(self, heads, dim, resident_pages, levels=2, dtype=torch.float32, device="cpu", path: Optional[str] = None):
        self.shape = (2, PAGE, heads, dim)
        self.page_elems = 2 * PAGE * heads * dim
        self.dtype, self.device = dtype, torch.device(device)
        self.fast = torch.zeros((resident_pages,) + self.shape, dtype=dtype, device=self.device)
        self.free = list(range(resident_pages - 1, -1, -1))
        self.table = PageTable(levels)                       # logical page -> fast slot (resident pages only)
        self.lru: "OrderedDict[int, int]" = OrderedDict()    # logical page -> slot, oldest first
        self.on_disk = set()
        self.path = path or os.path.join(tempfile.mkdtemp(prefix="tfb_kv_"), "kv.spill")
        self.file = open(self.path, "w+b")
        self.esize = torch.empty((), dtype=dtype).element_size()
        self.lock = threading.Condition()
        self.inflight = set()
        self.q: "queue.Queue" = queue.Queue()
        self.worker = threading.Thread(target=self._work, daemon=True)
        self.worker.start()
        self.stats = {"evictions": 0, "loads": 0, "hits": 0}

    # ---- disk
    def _write(self, lpn, data: torch.Tensor):
        self.file.seek(lpn * self.page_elems * self.esize)
        self.file.write(data.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes())
        self.file.flush()

    def _read(self, lpn) -> torch.Tensor:
        self.file.seek(lpn * self.page_elems * self.esize)
        raw = self.file.read(self.page_elems * self.esize)
        return torch.frombuffer(bytearray(raw), dtype=self.dtype).view(self.shape)

    def _work(self):
        while True:
            job = self.q.get()
            if job is None:
                return
            lpn = job
            data = self._read(lpn)
            with self.lock:
                slot = self._slot_locked()
                self.fast[slot].copy_(data)
                self.table.set(lpn, slot)
                self.lru[lpn] = slot
                self.inflight.discard(lpn)
                self.stats["loads"] += 1
                self.lock.notify_all()

    # ---- residency
    def _slot_locked(self) -> int:
        if self.free:
            return self.free.pop()
        victim, slot = self.lru.popitem(last=False)
        self._write(victim, self.fast[slot])
        self.on_disk.add(victim)
        self.table.pop(victim)
        self.stats["evictions"] += 1
        return slot

    def write_page(self, lpn, kv: torch.Tensor):
        with self.lock:
            slot = self.table.get(lpn)
            if slot is None:
                slot = self._slot_locked()
                self.table.set(lpn, slot)
            self.fast[slot].copy_(kv.to(self.dtype))
            self.lru[lpn] = slot
            self.lru.move_to_end(lpn)

    def prefetch(self, lpns):
        with self.lock:
            for l in lpns:
                if self.table.get(l) is None and l in self.on_disk and l not in self.inflight:
                    self.inflight.add(l)
                    self.q.put(l)

    def ensure_resident(self, lpns, timeout_ms=5000) -> bool:
        """Bring pages back from disk; False when they did not arrive within the timeout."""
        self.prefetch(lpns)
        end = time.time() + timeout_ms / 1e3
        with self.lock:
            while any(self.table.get(l) is None for l in lpns if l in self.on_disk or l in self.inflight):
                rest = end - time.time()
                if rest <= 0:
                    return False
                self.lock.wait(rest)
            for l in lpns:
                if l in self.lru:
                    self.lru.move_to_end(l)
                    self.stats["hits"] += 1
        return True

    def read_page(self, lpn) -> torch.Tensor:
        if not self.ensure_resident([lpn]):
            raise TimeoutError(f"page {lpn} did not become resident")
        with self.lock:
            return self.fast[self.table.get(lpn)].clone()

    def close(self):
        self.q.put(None)
        self.worker.join(timeout=2)
        self.file.close()


def PagedKVCache4M(heads, dim, resident_pages=1024, **kw):
    return TieredKVStore(heads, dim, resident_pages, levels=2, **kw)


def PagedKVCache1T(heads, dim, resident_pages=1024, **kw):
    return TieredKVStore(heads, dim, resident_pages, levels=3, **kw)


class CompressedKVCache:
    """Ternary K / V: per 32 elements one fp16 scale (mean |x|) and 2-bit codes {-1, 0, +1}."""

    def __init__(self, heads, dim, max_tokens, device="cpu"):
        assert dim % 32 == 0
        self.H, self.D = heads, dim
        self.codes = torch.zeros((2, max_tokens, heads, dim // 4), dtype=torch.uint8, device=device)
        self.scales = torch.zeros((2, max_tokens, heads, dim // 32), dtype=torch.float16, device=device)
        self.len = 0

    @staticmethod
    def _enc(x):
        g = x.float().reshape(*x.shape[:-1], -1, 32)
        s = g.abs().mean(-1, keepdim=True).clamp(min=1e-8)
        c = torch.where(g > 0.5 * s, 2, torch.where(g < -0.5 * s, 0, 1)).to(torch.uint8).reshape(*x.shape[:-1], -1, 4)
        packed = c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)
        return packed, s[..., 0].to(torch.float16)

    def append(self, k, v):
        n = k.shape[0]
        for i, t in enumerate((k, v)):
            p, s = self._enc(t)
            self.codes[i, self.len:self.len + n], self.scales[i, self.len:self.len + n] = p, s
        self.len += n

    def get(self):
        out = []
        for i in range(2):
            p = self.codes[i, : self.len]
            c = torch.stack([p & 3, (p >> 2) & 3, (p >> 4) & 3, p >> 6], -1).reshape(self.len, self.H, self.D).float() - 1
            out.append(c * self.scales[i, : self.len].float().repeat_interleave(32, -1))
        return out[0], out[1]

    def bytes_per_token(self):
        return 2 * self.H * (self.D / 4 + self.D / 32 * 2)

    def _row(self, i, pos):
        p = self.codes[i, pos]
        c = torch.stack([p & 3, (p >> 2) & 3, (p >> 4) & 3, p >> 6], -1).reshape(self.H, self.D).float() - 1
        return c * self.scales[i, pos].float().repeat_interleave(32, -1)

    def get_k(self, pos: int) -> torch.Tensor:
        """Decoded keys [heads, dim] of one cached position."""
        if not 0 <= pos < self.len:
            raise IndexError(pos)
        return self._row(0, pos)

    def get_v(self, pos: int) -> torch.Tensor:
        if not 0 <= pos < self.len:
            raise IndexError(pos)
        return self._row(1, pos)

    def size(self) -> int: return self.len

    def clear(self):
        self.len = 0


def flash_decoding(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, splits=4, scale=None):
    """q [H, D], k / v [N, Hkv, D] -> [H, D]; the key range is cut into ``splits`` chunks whose partial (max, sum, output)
    triples are merged with the log-sum-exp rule."""
    H, D = q.shape
    N, Hkv, _ = k.shape
    G = H // Hkv
    scale = scale or D ** -0.5
    qf = q.float().view(Hkv, G, D)
    parts = []
    for c in torch.arange(N).chunk(splits):
        if c.numel() == 0:
            continue
        s = torch.einsum("hgd,nhd->hgn", qf, k[c].float()) * scale
        m = s.amax(-1)
        p = torch.exp(s - m[..., None])
        parts.append((m, p.sum(-1), torch.einsum("hgn,nhd->hgd", p, v[c].float())))
    M = torch.stack([m for m, _, _ in parts]).amax(0)
    L = sum(l * torch.exp(m - M) for m, l, _ in parts)
    O = sum(o * torch.exp(m - M)[..., None] for m, _, o in parts)
    return (O / L[..., None]).reshape(H, D).to(q.dtype)


@dataclass
class ReasoningBudget:
    """Caps on hidden reasoning tokens before the visible answer must start."""
    LOW, MEDIUM, HIGH = 256, 2048, 8192
    budget: int = 2048
    used: int = 0

    @classmethod
    def for_level(cls, level: str):
        return cls({"low": cls.LOW, "medium": cls.MEDIUM, "high": cls.HIGH}[level])

    def consume(self, n=1) -> bool:
        """True while thinking may continue."""
        self.used += n
        return self.used < self.budget

    def remaining(self):
        return max(0, self.budget - self.used)


class PagedAttention:
    """alloc_block / free_block / forward over a ``PagedKVCache`` layer (block = 16-token page)."""

    def __init__(self, cache, layer=0):
        self.cache, self.layer = cache, layer

    def alloc_block(self) -> int:
        return self.cache.allocator.alloc()

    def free_block(self, block_id: int):
        self.cache.allocator.release(block_id)

    def num_blocks(self) -> int:
        """Pages of the pool (page 0 is the scratch page of padded rows)."""
        return len(self.cache.allocator.refs)

    def available_blocks(self) -> int:
        return len(self.cache.allocator.free)

    def forward(self, q, block_table, seq_lens, num_q_heads):
        return self.cache.decode(self.layer, q, block_table, seq_lens, num_q_heads)


@dataclass
class BatchRequest:
    tokens: List[int]
    max_tokens: int = 64
    id: int = 0


@dataclass
class BatchResponse:
    text: str
    id: int
    tokens: List[int]


class ContinuousBatching:
    def __init__(self, model, tokenizer=None, max_batch=8, **engine_kw):
        from .engine import EngineConfig, InferenceEngine
        self.tok = tokenizer
        self.engine = InferenceEngine(model, tokenizer, EngineConfig(max_batch=max_batch, **engine_kw))
        self.ids: Dict[int, int] = {}

    def add_request(self, req: BatchRequest, sampling=None):
        r = self.engine.add_request(req.tokens, req.max_tokens, sampling)
        self.ids[r.id] = req.id

    def has_pending(self):
        return self.engine.has_pending()

    def step(self) -> List[BatchResponse]:
        out = []
        for r in self.engine.step():
            text = self.tok.decode([t for t in r.out if t != getattr(self.tok, "eos_id", -1)]) if self.tok else ""
            out.append(BatchResponse(text, self.ids.pop(r.id, r.id), list(r.out)))
        return out


class Q4KVCache:
    """Per-layer key / value store quantised to 4 bits with a 16-entry fp16 codebook per block, trained for every block
    by Lloyd-Max (uniform start over the block's range, at most 20 assign / centroid rounds).  Blocks of ``block_size``
    (32 / 64 / 128) elements run over the flattened [token][head][dim] stream of one token chunk; indices are packed two
    per byte, low nibble first.  ``get_range`` returns fp32 [1, heads, length, dim].  The paged engine's own 4-bit mode
    (scale per 32 elements, ``PagedKVCache(kv_mode="q4")``) is the device form; this class keeps the reference's
    codebook form and its API.

    Reference counterpart: Q4KVCache (include/quant/kv_cache_quant4.h, src/model/kv_cache_quant4.cpp:77-152 training,
    :181-199 nibble order, :207-291 append, :293-362 get_range, :388 compression_ratio)."""
    Q4_CODEBOOK_SIZE = 16

    def __init__(self, num_layers: int, max_seq_len: int, num_heads: int, head_dim: int, block_size: int = 64, device="cpu"):
        assert block_size in (32, 64, 128)
        self.num_layers, self._max_seq_len, self.num_heads, self.head_dim, self._block = num_layers, max_seq_len, num_heads, head_dim, block_size
        self.device = torch.device(device)
        per_tok = num_heads * head_dim
        assert per_tok % block_size == 0, "heads x dim must be a whole number of blocks"
        self.blocks_per_token = per_tok // block_size
        nb = max_seq_len * self.blocks_per_token
        mk_i = lambda: torch.zeros((nb, block_size // 2), dtype=torch.uint8, device=self.device)
        mk_c = lambda: torch.zeros((nb, 16), dtype=torch.float16, device=self.device)
        self.k_idx, self.v_idx = [mk_i() for _ in range(num_layers)], [mk_i() for _ in range(num_layers)]
        self.k_cb, self.v_cb = [mk_c() for _ in range(num_layers)], [mk_c() for _ in range(num_layers)]
        self.pos = [0] * num_layers

    def init(self, num_layers: int, max_seq_len: int, num_heads: int, head_dim: int, block_size: int = 64):
        """Re-create the store with new dimensions; everything cached is dropped."""
        self.__init__(num_layers, max_seq_len, num_heads, head_dim, block_size, self.device)
        return self

    # ---- block codec (batched over blocks)
    @staticmethod
    def quantize_blocks(x: torch.Tensor, iters: int = 20):
        """x [nb, n] fp32 -> (packed indices uint8 [nb, n / 2], codebook fp16 [nb, 16])."""
        x = x.float()
        lo, hi = x.min(-1, keepdim=True).values, x.max(-1, keepdim=True).values
        span = (hi - lo).clamp(min=1e-12)
        cb = lo + span * (torch.arange(16, device=x.device, dtype=torch.float32)[None, :] + 0.5) / 16.0
        for _ in range(iters):
            idx = (x[:, :, None] - cb[:, None, :]).abs().argmin(-1)                      # [nb, n]
            onehot = torch.nn.functional.one_hot(idx, 16).float()
            cnt = onehot.sum(1)
            new = (onehot * x[:, :, None]).sum(1) / cnt.clamp(min=1)
            new = torch.where(cnt > 0, new, cb)                                         # empty cells keep their centre
            if torch.allclose(new, cb, atol=0, rtol=1e-6):
                cb = new
                break
            cb = new
        cb16 = cb.to(torch.float16)
        idx = (x[:, :, None] - cb16.float()[:, None, :]).abs().argmin(-1).to(torch.uint8)
        packed = idx[:, 0::2] | (idx[:, 1::2] << 4)
        return packed, cb16

    @staticmethod
    def dequantize_blocks(packed: torch.Tensor, cb16: torch.Tensor):
        idx = torch.stack([packed & 0xF, packed >> 4], -1).reshape(packed.shape[0], -1).long()
        return cb16.float().gather(1, idx)

    quantize_block_quant4 = quantize_blocks
    dequantize_block_quant4 = dequantize_blocks

    # ---- cache API
    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        """k, v: [1, heads, t, dim] (or [heads, t, dim]) for t new tokens of ``layer``."""
        k = k.reshape(self.num_heads, -1, self.head_dim)
        v = v.reshape(self.num_heads, -1, self.head_dim)
        t = k.shape[1]
        p0 = self.pos[layer]
        if p0 + t > self._max_seq_len:
            raise ValueError("Q4KVCache is full")
        for src, idx, cb in ((k, self.k_idx[layer], self.k_cb[layer]), (v, self.v_idx[layer], self.v_cb[layer])):
            flat = src.permute(1, 0, 2).reshape(t * self.blocks_per_token, self._block).to(self.device)   # [token][head][dim]
            pk, c16 = self.quantize_blocks(flat)
            b0 = p0 * self.blocks_per_token
            idx[b0:b0 + pk.shape[0]] = pk
            cb[b0:b0 + pk.shape[0]] = c16
        self.pos[layer] = p0 + t

    def get_range(self, layer: int, start: int, end: int):
        end = min(end, self.pos[layer])
        n = max(0, end - start)
        out = []
        for idx, cb in ((self.k_idx[layer], self.k_cb[layer]), (self.v_idx[layer], self.v_cb[layer])):
            b0, b1 = start * self.blocks_per_token, end * self.blocks_per_token
            x = self.dequantize_blocks(idx[b0:b1], cb[b0:b1]).reshape(n, self.num_heads, self.head_dim)
            out.append(x.permute(1, 0, 2).unsqueeze(0).contiguous())
        return out[0], out[1]

    def get_all(self, layer: int):
        return self.get_range(layer, 0, self.pos[layer])

    def context_len(self) -> int:
        return self.pos[0] if self.pos else 0

    def max_seq_len(self):
        return self._max_seq_len

    def block_size(self):
        return self._block

    def size_bytes(self) -> int:
        used = sum(self.pos) * self.blocks_per_token
        return 2 * used * (self._block // 2 + 32)

    def size_bytes_fp32_equivalent(self) -> int:
        return 2 * sum(self.pos) * self.num_heads * self.head_dim * 4

    def compression_ratio(self) -> float:
        return self.size_bytes_fp32_equivalent() / max(1, self.size_bytes())

    def clear(self):
        self.pos = [0] * self.num_layers

    def resize(self, new_max_seq_len: int):
        keep = min(new_max_seq_len, self._max_seq_len) * self.blocks_per_token
        for lst, width, dt in ((self.k_idx, self._block // 2, torch.uint8), (self.v_idx, self._block // 2, torch.uint8),
                               (self.k_cb, 16, torch.float16), (self.v_cb, 16, torch.float16)):
            for i, t in enumerate(lst):
                n = torch.zeros((new_max_seq_len * self.blocks_per_token, width), dtype=dt, device=self.device)
                n[:keep] = t[:keep]
                lst[i] = n
        self._max_seq_len = new_max_seq_len
        self.pos = [min(p, new_max_seq_len) for p in self.pos]
