"""Paged KV cache: a pool of 16-token pages per layer with bf16, fp8-e4m3 or 4-bit storage, a page
allocator with reference counts (prefix sharing), and the device operators that write new tokens
into their slots and run decode attention straight from the quantised pages.

Reference counterparts: PagedKVCacheBase (block_size 16, src/model/kv_cache.cpp:389-946), Q4KVCache
(src/model/kv_cache_quant4.cpp), KVCache "FP8" = int8 absmax (src/model/kv_cache.cpp:63-92; here real
E4M3), PagedAttention alloc_block/free_block (include/quant/inference_opt.h:17-90).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..ops import _lib
from ..ops._lib import c_f, c_i, c_ll, c_p, check, ptr, stream

PAGE = 16
MODES = {"bf16": 0, "fp8": 1, "q4": 2}

_lib.register("tfb_kv_append", [c_p, c_ll, c_i, c_i, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_ll, c_p])
_lib.register("tfb_kv_gather", [c_p, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_ll, c_i, c_i, c_i, c_ll, c_p])
_lib.register("tfb_paged_decode", [c_p, c_ll, c_p, c_p, c_p, c_p, c_p, c_i, c_p, c_p, c_ll, c_p, c_p, c_i, c_i, c_i,
                                   c_i, c_i, c_i, c_f, c_ll, c_p, c_p])


class PageAllocator:
    """Free-list page allocator with reference counts (a page shared by a cached prefix is freed when
    the last sequence using it lets go)."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free: List[int] = list(range(num_pages - 1, -1, -1))
        self.refs = [0] * num_pages

    def alloc(self) -> int:
        if not self.free:
            raise MemoryError("KV cache is out of pages")
        p = self.free.pop()
        self.refs[p] = 1
        return p

    def share(self, page: int):
        self.refs[page] += 1

    def release(self, page: int):
        self.refs[page] -= 1
        if self.refs[page] == 0:
            self.free.append(page)

    @property
    def num_free(self):
        return len(self.free)


class _Pool:
    def __init__(self, pages, Hkv, D, mode, device):
        self.mode = mode
        if mode == "bf16":
            self.data = torch.zeros((pages, PAGE, Hkv, D), dtype=torch.bfloat16, device=device)
            self.scale = None
        elif mode == "fp8":
            self.data = torch.zeros((pages, PAGE, Hkv, D), dtype=torch.uint8, device=device)
            self.scale = torch.ones((pages, PAGE, Hkv), dtype=torch.float32, device=device)
        elif mode == "q4":
            self.data = torch.full((pages, PAGE, Hkv, D // 2), 0x88, dtype=torch.uint8, device=device)
            self.scale = torch.ones((pages, PAGE, Hkv, D // 32), dtype=torch.float16, device=device)
        else:
            raise ValueError(mode)

    def dequant(self):
        """fp32 [pages, 16, Hkv, D] (oracle / CPU path)."""
        if self.mode == "bf16":
            return self.data.float()
        if self.mode == "fp8":
            return self.data.view(torch.float8_e4m3fn).float() * self.scale[..., None]
        lo = (self.data & 15).float() - 8
        hi = (self.data >> 4).float() - 8
        v = torch.stack([lo, hi], -1).flatten(-2)
        return v * self.scale.float().repeat_interleave(32, -1)

    def write_ref(self, slots, rows):
        """CPU statement of kv_append for rows [n, Hkv, D] at flat slot indices."""
        pages, sl = slots // PAGE, slots % PAGE
        r = rows.float()
        if self.mode == "bf16":
            self.data[pages, sl] = r.to(torch.bfloat16)
        elif self.mode == "fp8":
            amax = r.abs().amax(-1)
            s = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
            self.scale[pages, sl] = s
            self.data[pages, sl] = (r / s[..., None]).to(torch.float8_e4m3fn).view(torch.uint8)
        else:
            n, H, D = r.shape
            blk = r.view(n, H, D // 32, 32)
            amax = blk.abs().amax(-1)
            s = torch.where(amax > 0, amax / 7.0, torch.ones_like(amax)).to(torch.float16)
            self.scale[pages, sl] = s
            q = (torch.round(blk / s.float()[..., None]) + 8).clamp(0, 15).to(torch.uint8).view(n, H, D)
            self.data[pages, sl] = q[..., 0::2] | (q[..., 1::2] << 4)


class PagedKVCache:
    """KV pools of every layer of one model shard."""

    def __init__(self, num_layers, num_pages, Hkv, D, mode="bf16", device="cuda"):
        assert mode in MODES
        if torch.device(device).type == "cuda":
            assert D in (64, 128), "the paged-attention kernels are built for head_dim 64 and 128"
        else:
            assert D % 32 == 0 or mode != "q4", "4-bit KV blocks hold 32 elements"
        self.L, self.num_pages, self.Hkv, self.D, self.mode = num_layers, num_pages, Hkv, D, mode
        self.device = torch.device(device)
        self.k = [_Pool(num_pages, Hkv, D, mode, device) for _ in range(num_layers)]
        self.v = [_Pool(num_pages, Hkv, D, mode, device) for _ in range(num_layers)]
        self.allocator = PageAllocator(num_pages)
        self._ws = {}

    @classmethod
    def init(cls, num_layers: int, max_seq_len: int, num_heads: int, head_dim: int, mode="bf16", device="cuda", sequences: int = 1):
        """A cache with room for ``sequences`` sequences of ``max_seq_len`` tokens (rounded up to whole pages)."""
        return cls(num_layers, sequences * ((max_seq_len + PAGE - 1) // PAGE), num_heads, head_dim, mode, device)

    def logical_capacity(self) -> int:
        """Tokens the pools can hold over all sequences."""
        return self.num_pages * PAGE

    def max_seq_len(self) -> int:
        """The longest single sequence: one that owns every page."""
        return self.num_pages * PAGE

    def bytes_per_token(self) -> float:
        per = {"bf16": 2.0, "fp8": 1.0 + 4.0 / self.D, "q4": 0.5 + 2.0 / 32}[self.mode]
        return 2 * self.L * self.Hkv * self.D * per

    def append(self, layer, src, k_col0, v_col0, slot_mapping):
        """Write the K / V rows of ``src`` [T, ld] (bf16, post-RoPE) into flat slots (page*16 + offset)."""
        kp, vp = self.k[layer], self.v[layer]
        T = src.shape[0]
        if not src.is_cuda:
            keep = slot_mapping >= 0
            H, D = self.Hkv, self.D
            kp.write_ref(slot_mapping[keep], src[keep, k_col0:k_col0 + H * D].reshape(-1, H, D))
            vp.write_ref(slot_mapping[keep], src[keep, v_col0:v_col0 + H * D].reshape(-1, H, D))
            return
        check(_lib.lib().tfb_kv_append(src.data_ptr(), src.stride(0), k_col0, v_col0, slot_mapping.data_ptr(),
                                       kp.data.data_ptr(), ptr(kp.scale), vp.data.data_ptr(), ptr(vp.scale), T,
                                       self.Hkv, self.D, MODES[self.mode], self.num_pages * PAGE, stream()), "kv_append")

    def gather(self, layer, pages, n):
        """The first ``n`` cached tokens of one sequence (``pages``: its page list, int32 tensor) as contiguous bf16 rows
        (k [n, Hkv*D], v [n, Hkv*D]), dequantised: the keys / values a prompt suffix attends over besides itself."""
        kp, vp = self.k[layer], self.v[layer]
        Hkv, D = self.Hkv, self.D
        if not kp.data.is_cuda:
            K, V = kp.dequant(), vp.dequant()
            pg = pages[: (n + PAGE - 1) // PAGE].long()
            return (K[pg].reshape(-1, Hkv * D)[:n].to(torch.bfloat16), V[pg].reshape(-1, Hkv * D)[:n].to(torch.bfloat16))
        ok = torch.empty((n, Hkv * D), dtype=torch.bfloat16, device=kp.data.device)
        ov = torch.empty_like(ok)
        check(_lib.lib().tfb_kv_gather(kp.data.data_ptr(), ptr(kp.scale), vp.data.data_ptr(), ptr(vp.scale), pages.data_ptr(), n,
                                       ok.data_ptr(), ov.data_ptr(), Hkv * D, Hkv, D, MODES[self.mode], self.num_pages * PAGE,
                                       stream()), "kv_gather")
        return ok, ov

    def decode(self, layer, q, block_table, seq_lens, Hq, scale=None, splits=None):
        """q [B, Hq*D] bf16 -> o [B, Hq*D] attending over the first seq_lens[b] cached tokens of each sequence."""
        B = q.shape[0]
        D, Hkv = self.D, self.Hkv
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        if not q.is_cuda:
            K, V = self.k[layer].dequant(), self.v[layer].dequant()
            out = torch.zeros(B, Hq * D)
            G = Hq // Hkv
            for b in range(B):
                n = int(seq_lens[b])
                pages = block_table[b, : (n + PAGE - 1) // PAGE].long()
                kk = K[pages].reshape(-1, Hkv, D)[:n]
                vv = V[pages].reshape(-1, Hkv, D)[:n]
                qq = q[b].float().view(Hkv, G, D)
                s = torch.einsum("hgd,nhd->hgn", qq, kk) * scale
                out[b] = torch.einsum("hgn,nhd->hgd", torch.softmax(s, -1), vv).reshape(-1)
            return out.to(q.dtype)
        if splits is None:
            max_len = block_table.shape[1] * PAGE
            # enough CTAs (128 threads each) for about eight per SM: the kernel is latency-bound per CTA (one K row per
            # thread, then a serial walk over the tile's V rows), so parallelism across CTAs is what hides it
            splits = max(1, min(16, (8 * 148) // max(1, B * Hkv), max_len // 128))
        key = (B, Hq, splits)
        if key not in self._ws:
            self._ws[key] = (torch.empty(B * Hq * splits * D, dtype=torch.float32, device=q.device),
                             torch.empty(B * Hq * splits * 2, dtype=torch.float32, device=q.device))
        acc, ml = self._ws[key]
        o = torch.empty((B, Hq * D), dtype=q.dtype, device=q.device)
        kp, vp = self.k[layer], self.v[layer]
        check(_lib.lib().tfb_paged_decode(q.data_ptr(), q.stride(0), kp.data.data_ptr(), ptr(kp.scale),
                                          vp.data.data_ptr(), ptr(vp.scale), block_table.data_ptr(),
                                          block_table.shape[1], seq_lens.data_ptr(), o.data_ptr(), o.stride(0),
                                          acc.data_ptr(), ml.data_ptr(), B, Hq, Hkv, D, splits, MODES[self.mode],
                                          float(scale), self.num_pages * PAGE, _lib.status_word(q.device).data_ptr(),
                                          stream()), "paged_decode", 2)
        return o
