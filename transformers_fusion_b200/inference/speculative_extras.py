"""Pieces around speculative decoding and inference memory that stand on their own: the speed-up model that picks the
draft length, batch verification of draft positions, KV checkpoints for rewinding rejected drafts, a byte-budgeted
request memory pool, tiled attention for very long contexts (full and local-window), and a per-process GPU inventory.

Reference counterparts: Theorem13Result / SmallBatchVerifier / KVCheckpoint (include/quant/speculative_decoder.h:47-53,
129-180; src/inference/speculative_decoder.cpp:193-250), InferenceMemoryPool (src/inference/inference_paging.cpp:122-285),
MemoryEfficientAttention forward / forward_block_sparse, max_context_tokens 4M (src/trainer/zero_optimizer_mem.cpp:179-494),
MultiGPUManager detect / allocate_on / transfer (src/backend/gpu_extras.cpp:154-455)."""
from __future__ import annotations

import threading

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch


# ------------------------------------------------------------------------------------------------ draft-length model
@dataclass
class SpeculationPlan:
    """Expected speed-up S(k, a) = (1 + k a) / (1 + k c) of drafting k tokens with acceptance rate a when a draft step
    costs c target steps; k* = round(sqrt(2 / (1 - a))) when a > c, otherwise speculation does not pay (k = 1, S = 1)."""
    speedup: float = 1.0
    optimal_k: int = 1
    acceptance_rate: float = 0.0
    cost_ratio: float = 0.0

    @staticmethod
    def compute(alpha: float, cost_ratio: float) -> "SpeculationPlan":
        r = SpeculationPlan(1.0, 1, alpha, cost_ratio)
        if alpha <= cost_ratio:
            return r
        r.optimal_k = max(1, round(math.sqrt(2.0 / max(1e-9, 1.0 - alpha))))
        r.speedup = (1.0 + r.optimal_k * alpha) / (1.0 + r.optimal_k * cost_ratio)
        return r


Theorem13Result = SpeculationPlan


@dataclass
class VerificationResult:
    accepted: List[bool] = field(default_factory=list)
    first_rejection_pos: int = -1
    total_accepted: int = 0
    verify_flops: float = 0.0
    verify_inferno: float = 0.0          # the comparison work weighted by the information weight of the weight format


class SmallBatchVerifier:
    """Greedy verification of up to ``max_batch`` draft positions in one pass: position i is accepted while the draft's
    arg-max equals the target's; everything after the first mismatch is rejected."""

    def __init__(self, max_batch: int = 8):
        self.max_batch = max_batch
        self.format_index = 5            # Q_8 in the throughput counter's format table

    def set_format_index(self, idx: int):
        """Which weight format the verified model runs in (index into ``InfernoCounter.FORMATS``): it sets the information
        weight applied to ``verify_flops`` in the result's ``verify_inferno``."""
        self.format_index = int(idx)

    def verify(self, draft_logits: torch.Tensor, target_logits: torch.Tensor, temperature: float = 1.0) -> VerificationResult:
        n = min(self.max_batch, draft_logits.shape[0], target_logits.shape[0])
        res = VerificationResult([False] * n, n, 0, 2.0 * n)
        if n == 0 or draft_logits.shape[-1] != target_logits.shape[-1]:
            res.first_rejection_pos = 0 if n else -1
            return res
        from ..utils.inferno import InfernoCounter
        if 0 <= self.format_index < len(InfernoCounter.FORMATS):
            res.verify_inferno = res.verify_flops * (32.0 / InfernoCounter.FORMATS[self.format_index][1]) / 2.0
        same = (draft_logits[:n].argmax(-1) == target_logits[:n].argmax(-1)).tolist()
        for i, ok in enumerate(same):
            if not ok:
                res.first_rejection_pos = i
                break
            res.accepted[i] = True
            res.total_accepted += 1
        return res


@dataclass
class KVCheckpoint:
    """Length (and page count) of one sequence in the paged cache at the moment drafting started."""
    seq_len: int = 0
    num_pages: int = 0
    valid: bool = False


def checkpoint_kv(pages: Sequence[int], seq_len: int) -> KVCheckpoint:
    return KVCheckpoint(seq_len, len(pages), True)


def rewind_kv(allocator, pages: List[int], ckpt: KVCheckpoint, new_len: int, page_size: int = 16) -> int:
    """Drops the cache entries past ``new_len`` (>= the checkpointed length is allowed: accepted draft tokens stay): pages
    that are no longer needed go back to the allocator.  Entries inside the last kept page are simply overwritten by the
    next append.  Returns the new length."""
    if not ckpt.valid:
        raise ValueError("invalid KV checkpoint")
    new_len = max(new_len, 0)
    keep = max((new_len + page_size - 1) // page_size, min(ckpt.num_pages, (ckpt.seq_len + page_size - 1) // page_size) if new_len >= ckpt.seq_len else 0)
    keep = max(keep, (new_len + page_size - 1) // page_size)
    while len(pages) > keep:
        allocator.release(pages.pop())
    return new_len


# ------------------------------------------------------------------------------------------------ memory pool
class InferenceMemoryPool:
    """Byte-budgeted bookkeeping of per-request memory (KV pages, scratch).  ``reserve`` fails rather than overcommits;
    the scheduler admits a request only when its worst case fits."""

    def __init__(self, capacity_bytes: int):
        self.capacity, self.used = int(capacity_bytes), 0
        self._by_owner: Dict[object, int] = {}
        self.peak = 0
        self._lock = threading.Lock()

    def reserve(self, owner, nbytes: int) -> bool:
        if nbytes < 0 or self.used + nbytes > self.capacity:
            return False
        self._by_owner[owner] = self._by_owner.get(owner, 0) + nbytes
        self.used += nbytes
        self.peak = max(self.peak, self.used)
        return True

    def release(self, owner) -> int:
        n = self._by_owner.pop(owner, 0)
        self.used -= n
        return n

    # ---- fixed-size block form (reference: InferenceMemoryPool(block_size, num_blocks), include/quant/inference_opt.h:188-201)
    @classmethod
    def of_blocks(cls, block_size: int, num_blocks: int) -> "InferenceMemoryPool":
        pool = cls(block_size * num_blocks)
        pool.block_size, pool._free_blocks = block_size, list(range(num_blocks - 1, -1, -1))
        return pool

    def alloc(self):
        """Handle (block index) of a free block, or None when the pool is exhausted."""
        free = getattr(self, "_free_blocks", None)
        if free is None:
            raise RuntimeError("alloc() needs a pool made with InferenceMemoryPool.of_blocks")
        with self._lock:
            if not free:
                return None
            self.used += self.block_size
            return free.pop()

    def free(self, handle: int):
        with self._lock:
            if handle in self._free_blocks:
                raise ValueError(f"block {handle} is already free")
            self._free_blocks.append(handle)
            self.used -= self.block_size

    def available(self) -> int: return self.capacity - self.used
    def utilization(self) -> float: return self.used / self.capacity if self.capacity else 0.0
    def owners(self) -> int: return len(self._by_owner)


# ------------------------------------------------------------------------------------------------ long-context attention
class MemoryEfficientAttention:
    """Exact attention computed in (block_q x block_k) tiles with a running max / sum, so memory is O(S * d) instead of
    O(S^2); ``forward_block_sparse`` restricts every query to the keys inside a local window (and optional global
    prefix).  This is the host / oracle statement; the device path of the framework is the flash-attention kernel."""

    def __init__(self, block_q: int = 64, block_k: int = 64, max_context_tokens: int = 4 << 20):
        self.bq, self.bk, self.max_context_tokens = block_q, block_k, max_context_tokens

    def _run(self, q, k, v, causal, window, n_global, mask):
        S, Sk, d = q.shape[-2], k.shape[-2], q.shape[-1]
        if not torch.is_grad_enabled():
            self._stats = {"max_val": -float("inf"), "sum_val": 0.0, "num_blocks": 0}
        if max(S, Sk) > self.max_context_tokens:
            raise ValueError(f"context of {max(S, Sk)} tokens exceeds the limit of {self.max_context_tokens}")
        scale = 1.0 / math.sqrt(d)
        out = torch.zeros_like(q, dtype=torch.float32)
        qpos_all, kpos_all = torch.arange(S, device=q.device), torch.arange(Sk, device=q.device)
        for q0 in range(0, S, self.bq):
            qb = q[..., q0:q0 + self.bq, :].float()
            qpos = qpos_all[q0:q0 + self.bq] + (Sk - S)            # queries are the last S positions of the keys
            m = torch.full(qb.shape[:-1], -float("inf"), device=q.device)
            l = torch.zeros(qb.shape[:-1], device=q.device)
            acc = torch.zeros_like(qb)
            lo = 0 if window <= 0 else max(0, int(qpos[0]) - window + 1)
            hi = Sk if not causal else min(Sk, int(qpos[-1]) + 1)
            a0 = lo // self.bk * self.bk
            ranges = [(a0, hi)]
            if window > 0 and n_global > 0 and a0 > 0:
                ranges.insert(0, (0, min(n_global, a0)))
            for a, b in ranges:
                for k0 in range(a, b, self.bk):
                    k1 = min(k0 + self.bk, b)
                    kp = kpos_all[k0:k1]
                    s = qb @ k[..., k0:k1, :].float().transpose(-1, -2) * scale
                    ok = torch.ones((qpos.numel(), kp.numel()), dtype=torch.bool, device=q.device)
                    if causal:
                        ok &= kp[None, :] <= qpos[:, None]
                    if window > 0:
                        ok &= (kp[None, :] > qpos[:, None] - window) | (kp[None, :] < n_global)
                    if mask is not None:
                        ok &= mask[q0:q0 + self.bq, k0:k1]
                    s = s.masked_fill(~ok, -float("inf"))
                    m_new = torch.maximum(m, s.amax(-1))
                    safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
                    p = torch.exp(s - safe[..., None])
                    corr = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, -float("inf")), m) - safe)
                    l = l * corr + p.sum(-1)
                    acc = acc * corr[..., None] + p @ v[..., k0:k1, :].float()
                    m = m_new
            out[..., q0:q0 + self.bq, :] = acc / l.clamp(min=1e-30)[..., None]
            if not torch.is_grad_enabled():
                st = self.__dict__.setdefault("_stats", {"max_val": -float("inf"), "sum_val": 0.0, "num_blocks": 0})
                st["max_val"] = max(st["max_val"], float(m[torch.isfinite(m)].max()) if torch.isfinite(m).any() else st["max_val"])
                st["sum_val"] = float(l.mean())
                st["num_blocks"] += sum(-(-(b - a) // self.bk) for a, b in ranges)
        return out.to(q.dtype)

    def forward(self, q, k, v, causal: bool = True, mask: Optional[torch.Tensor] = None):
        return self._run(q, k, v, causal, 0, 0, mask)

    def forward_block_sparse(self, q, k, v, window: int = 1024, n_global: int = 0, causal: bool = True):
        return self._run(q, k, v, causal, window, n_global, None)

    # ---- backward, statistics and estimates (reference: MemoryEfficientAttention, include/quant/zero_optimizer.h:274-350)
    def config(self) -> dict:
        return {"block_size_q": self.bq, "block_size_kv": self.bk, "max_context_tokens": self.max_context_tokens}

    def set_config(self, block_size_q: Optional[int] = None, block_size_kv: Optional[int] = None, max_context_tokens: Optional[int] = None):
        self.bq, self.bk = block_size_q or self.bq, block_size_kv or self.bk
        self.max_context_tokens = max_context_tokens or self.max_context_tokens

    def backward(self, grad_output, q, k, v, causal: bool = True, mask: Optional[torch.Tensor] = None):
        """(dq, dk, dv) by recomputation: the forward is run again tile by tile under autograd (nothing of the first
        forward pass is kept), so the memory stays O(S * d)."""
        qd, kd, vd = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        with torch.enable_grad():
            out = self._run(qd, kd, vd, causal, 0, 0, mask)
        dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), grad_output.float())
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)

    @staticmethod
    def online_softmax_tile(scores, row_max, row_sum, output, v_tile):
        """One tile of the running soft-max: ``scores`` [rows, keys] of a key block and its values ``v_tile`` [keys, d]
        are folded into the running (row_max, row_sum, unnormalised output); returns the three updated tensors."""
        m_new = torch.maximum(row_max, scores.amax(-1))
        p = torch.exp(scores - m_new[..., None])
        corr = torch.exp(row_max - m_new)
        return m_new, row_sum * corr + p.sum(-1), output * corr[..., None] + p @ v_tile

    def last_softmax_stats(self) -> dict:
        """{max_val, sum_val, num_blocks} of the most recent forward (largest row maximum, mean row sum, key tiles visited)."""
        return dict(getattr(self, "_stats", {"max_val": 0.0, "sum_val": 0.0, "num_blocks": 0}))

    def forward_memory_bytes(self, B: int, H: int, N: int, D: int, dtype_bytes: int = 2) -> int:
        return B * self.memory_bytes(N, H, D, dtype_bytes)["tiled"]

    def backward_memory_bytes(self, B: int, H: int, N: int, D: int, dtype_bytes: int = 2) -> int:
        """Recomputation keeps the inputs, their gradients and one tile's intermediates twice (forward + its adjoint)."""
        return B * H * (6 * N * D * max(dtype_bytes, 4) + 2 * (self.bq * self.bk * 4 + self.bq * D * 4))

    def memory_bytes(self, seq: int, heads: int, dim: int, dtype_bytes: int = 2) -> Dict[str, int]:
        """Working set of the tiled form against the naive score matrix."""
        return {"tiled": heads * (self.bq * self.bk * 4 + self.bq * dim * 4 + 3 * seq * dim * dtype_bytes),
                "naive": heads * (seq * seq * 4 + 3 * seq * dim * dtype_bytes)}


# ------------------------------------------------------------------------------------------------ GPU inventory
@dataclass
class GPUInfo:
    index: int
    name: str
    total_bytes: int
    free_bytes: int
    sm_count: int
    capability: tuple


class MultiGPUManager:
    """What this process can see: devices, memory, and plain placement / copies between them.  Peer copies between GPUs of
    one node go over NVLink when peer access is available (``can_access_peer``)."""

    def detect(self) -> List[GPUInfo]:
        out = []
        if not torch.cuda.is_available():
            return out
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            free, total = torch.cuda.mem_get_info(i)
            out.append(GPUInfo(i, p.name, total, free, p.multi_processor_count, (p.major, p.minor)))
        return out

    def device_count(self) -> int:
        return torch.cuda.device_count() if torch.cuda.is_available() else 0

    def allocate_on(self, index: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        dev = torch.device("cuda", index) if self.device_count() else torch.device("cpu")
        return torch.empty(shape, dtype=dtype, device=dev)

    def transfer(self, t: torch.Tensor, index: int, non_blocking: bool = True) -> torch.Tensor:
        dev = torch.device("cuda", index) if self.device_count() else torch.device("cpu")
        return t.to(dev, non_blocking=non_blocking)

    # ---- the reference's verbs (include/quant/gpu_extras.h:63-77)
    def detect_devices(self) -> int:
        self._devices = self.detect()
        return len(self._devices)

    def init_device(self, index: int) -> bool:
        """Create the CUDA context of a device (a 1-element allocation does it); False for an index that does not exist."""
        if not 0 <= index < self.device_count():
            return False
        torch.empty(1, device=torch.device("cuda", index))
        if not hasattr(self, "_ready"):
            self._ready = set()
        self._ready.add(index)
        return True

    def device_name(self, index: int) -> str:
        return torch.cuda.get_device_properties(index).name if 0 <= index < self.device_count() else "cpu"

    def free_on(self, index: int, t: Optional[torch.Tensor] = None):
        """Drop a tensor's storage and hand cached blocks of that device back to the driver."""
        if t is not None:
            t.set_(torch.empty(0, dtype=t.dtype, device=t.device).untyped_storage(), 0, (0,))
        if 0 <= index < self.device_count():
            with torch.cuda.device(index):
                torch.cuda.empty_cache()

    def can_access_peer(self, a: int, b: int) -> bool:
        return self.device_count() > max(a, b) and (a == b or torch.cuda.can_device_access_peer(a, b))

    def least_loaded(self) -> int:
        infos = self.detect()
        return max(infos, key=lambda g: g.free_bytes).index if infos else -1
