"""Inference engine: paged KV cache, continuous batching, prefix reuse, priority scheduling, streaming.

One ``step()`` = admit waiting requests while pages are available (prefill each prompt with the
tcgen05 flash-attention kernel and scatter its K/V into pages, quantised on the way), then ONE decode
token for every running sequence in a single batched pass (GEMMs with M = batch, RoPE at per-sequence
positions, append to pages, paged decode attention on the tensor cores with fused KV dequantisation,
sampling kernel).  On CUDA the step is pipelined: the sampled ids stay on the device and feed the next
step there, which is launched before the host has read them (one step late, from a pinned buffer).
Finished sequences release their pages; a prefix cache lets requests that share a prompt prefix (whole
pages) reuse the pages instead of recomputing them, and the rest of such a prompt attends over the
cached pages through a gather + the tensor-core attention kernel.

Reference counterparts: ContinuousBatching / RequestScheduler (priority desc, deadline asc) /
PrefixCache / PagedAttention (src/inference/inference_paging.cpp:24-285, inference_kv.cpp:20-205),
Generator / StreamingGenerator events START / TOKEN / COMPLETE / STOP (src/inference/generator.cpp),
engine::InferenceEngine generate / generate_with_stats / generate_stream / generate_batch
(engines/inference/inference.h).
"""
from __future__ import annotations

import heapq
import itertools
import math
import time
import weakref
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from ..models.dense import _norm_fwd
from ..ops import functional as F
from .kv_cache import PAGE, PagedKVCache
from .sampler import SamplerConfig, sample


@dataclass
class EngineConfig:
    max_batch: int = 64
    num_pages: int = 4096
    kv_mode: str = "bf16"          # bf16 | fp8 | q4
    max_seq_len: int = 0           # 0 -> model config
    enable_prefix_cache: bool = True
    seed: int = 42
    weight_format: str = ""        # "" = bf16 weights; int8 | int4 | mxfp8 | fp4 | ternary: fused-dequant GEMM (quant/wq.py)
    weight_group: int = 32
    cuda_graph: bool = True        # decode steps replay a captured graph per batch-size bucket (CUDA only)
    batch_prefill: bool = True     # prompts admitted in the same step (without a cached prefix) are prefilled together
    max_prefill_tokens: int = 8192 # padded tokens per prefill batch
    pipeline_decode: object = True # CUDA: a decode step is launched before the previous step's tokens are read on the host
                                   # ("force": the same schedule on any device, for testing the scheduler on CPU)


@dataclass
class Request:
    tokens: List[int]
    max_tokens: int = 64
    sampling: SamplerConfig = field(default_factory=SamplerConfig)
    id: int = 0
    priority: int = 0
    deadline: float = float("inf")
    stop_ids: tuple = ()
    on_token: Optional[Callable[[int], None]] = None
    # runtime state
    out: List[int] = field(default_factory=list)
    pages: List[int] = field(default_factory=list)
    pos: int = 0
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    finished: bool = False


@dataclass
class InferenceStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    ttft_ms: float = 0.0
    tokens_per_sec: float = 0.0
    prefix_hit_tokens: int = 0


class PrefixCache:
    """Maps the hash of every whole-page token prefix to the page that holds its K/V."""

    def __init__(self, allocator):
        self.alloc = allocator
        self.table: Dict[int, int] = {}

    @staticmethod
    def _key(tokens, n):
        return hash(tuple(tokens[:n]))

    def lookup(self, tokens):
        pages = []
        n = PAGE
        while n <= len(tokens) - 1:   # at least one token must remain to produce logits
            p = self.table.get(self._key(tokens, n))
            if p is None or self.alloc.refs[p] == 0:
                break
            pages.append(p)
            n += PAGE
        for p in pages:
            self.alloc.share(p)
        return pages

    def insert(self, tokens, pages):
        for i, p in enumerate(pages):
            n = (i + 1) * PAGE
            if n > len(tokens):
                break
            k = self._key(tokens, n)
            if k not in self.table:
                self.table[k] = p
                self.alloc.share(p)    # the cache holds its own reference

    def evict_all(self):
        for p in self.table.values():
            self.alloc.release(p)
        self.table.clear()

    # ---- the reference's verbs (include/quant/inference_opt.h:108-119)
    def match_prefix(self, tokens) -> int:
        """Number of leading tokens whose K/V is cached (a multiple of the page size); takes no reference."""
        n = 0
        while n + PAGE <= len(tokens) - 1:
            p = self.table.get(self._key(tokens, n + PAGE))
            if p is None or self.alloc.refs[p] == 0:
                break
            n += PAGE
        return n

    def store(self, tokens, pages):
        """Remember the pages that hold the whole-page prefixes of ``tokens`` (same as ``insert``)."""
        self.insert(tokens, pages)

    def get_cache(self, tokens):
        """Pages of the longest cached prefix, each with a new reference for the caller (same as ``lookup``)."""
        return self.lookup(tokens)


class _TokenBuffers(list):
    """A claimed pair of pinned buffers; when the engine that holds it goes away the pair is free for the next engine."""


_PINNED_TOKENS: Dict[int, list] = {}        # device index -> [(weak reference to the claiming _TokenBuffers, [buf, buf])]


def _pinned_token_buffers(dev, n: int) -> _TokenBuffers:
    """Two pinned int64 buffers of at least n entries for the device -> host copy of a step's sampled ids.  The memory is
    kept for the life of the process and handed from engine to engine instead of being freed: a pinned block pending
    release makes the host allocator record and query events, and such calls disturb a stream capture in progress."""
    pool = _PINNED_TOKENS.setdefault(dev.index if dev.index is not None else torch.cuda.current_device(), [])
    for i, (owner, bufs) in enumerate(pool):
        if owner() is None and bufs[0].numel() >= n:
            break
    else:
        i, bufs = len(pool), [torch.empty(max(n, 64), dtype=torch.int64).pin_memory() for _ in range(2)]
        pool.append(None)
    held = _TokenBuffers(bufs)
    pool[i] = (weakref.ref(held), bufs)
    return held


class _DecodeGraph:
    """One captured decode step (all layers + final norm + LM head) for a fixed batch-size bucket.  Inputs live in static
    device buffers that the scheduler fills before each replay; rows past the live batch carry slot -1 (no KV write)
    and attend to one token of page 0, and their logits are ignored."""

    def __init__(self, eng, bucket: int):
        dev = eng.device
        self.bucket = bucket
        self.tokens = torch.zeros(bucket, dtype=torch.int64, device=dev)
        self.positions = torch.zeros(bucket, dtype=torch.int32, device=dev)
        self.bt = torch.zeros((bucket, eng.max_pages), dtype=torch.int32, device=dev)
        self.slots = torch.full((bucket,), -1, dtype=torch.int64, device=dev)
        run = lambda: eng._logits(eng._layers_decode(self.tokens, self.positions, self.bt, self.slots))
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                  # warm-up outside capture: workspaces, status words, lazy tables
            for _ in range(2):
                run()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        self._last_n = -1
        self.eng = eng
        self.token = eng._graph_capture_begin()
        # "relaxed": API calls that a capture in the default (global) mode forbids process-wide - an event query or a free by
        # the pinned-memory allocator on any thread, for instance, once pinned buffers of an earlier engine are pending
        # release - would invalidate the capture; nothing captured here depends on them
        with torch.cuda.graph(self.graph, capture_error_mode="relaxed"):
            self.logits = run()
            eng._graph_capture_end(self.token)

    def replay(self, tokens, positions, bt, slots):
        n = tokens.shape[0]
        self.tokens[:n].copy_(tokens, non_blocking=True)
        self.positions[:n].copy_(positions, non_blocking=True)
        self.bt[:n].copy_(bt, non_blocking=True)
        self.slots[:n].copy_(slots, non_blocking=True)
        if n < self.bucket and n != self._last_n:      # rows past the live batch: reset once per batch size
            self.positions[n:].zero_()
            self.slots[n:].fill_(-1)
        self._last_n = n
        self.eng._graph_before_replay(self.token)
        self.graph.replay()
        return self.logits[:n]


class InferenceEngine:
    def __init__(self, model, tokenizer=None, cfg: EngineConfig = EngineConfig()):
        self.model, self.tok, self.cfg = model, tokenizer, cfg
        mc = model.cfg
        self.device = model.tok_embeddings.device
        self.max_len = cfg.max_seq_len or mc.max_seq_len
        self.cache = PagedKVCache(mc.num_layers, cfg.num_pages, mc.num_kv_heads, mc.head_dim, cfg.kv_mode, self.device)
        self.prefix = PrefixCache(self.cache.allocator) if cfg.enable_prefix_cache else None
        self.waiting: list = []
        self.running: List[Request] = []
        self._ids = itertools.count(1)
        self._step = 0
        self._graphs = {}
        self._sample_cache = None
        self._bt_cache = None
        self._inflight = None          # (requests, device tokens, pinned host tokens, event) of the decode step in flight
        self._tok_host = None
        self.stats = InferenceStats()
        self.max_pages = (self.max_len + PAGE - 1) // PAGE
        self.packed = {}
        if cfg.weight_format:
            from ..quant import wq
            self._wq = wq
            self.packed = wq.quantize_model_linears(model, cfg.weight_format, cfg.weight_group, min_numel=0)

    # hooks around decode-graph capture and replay (the tensor-parallel engine keeps its collectives' host-side state
    # consistent with what a graph has baked in)
    def _graph_capture_begin(self):
        return None

    def _graph_capture_end(self, token):
        pass

    def _graph_before_replay(self, token):
        pass

    def _lin(self, x, li, name, w, bias=None, residual=None):
        """x @ W^T (+ bias) (+ residual) with W either the bf16 parameter or its packed low-bit form."""
        pw = self.packed.get(f"layers.{li}.{name}")
        if pw is None:
            return F.gemm(x, w.data, bias=bias, residual=residual)
        y = self._wq.gemm_wq(x, pw, bias)
        return y if residual is None else y + residual

    def _ffn(self, li, w, f, base):
        """Feed-forward half of a block on normed rows ``f`` with residual ``base``: the dense GLU / MLP, or - for a
        mixture-of-experts block - router, top-k dispatch, grouped expert GEMMs and weighted combine."""
        mc = self.model.cfg
        if hasattr(w, "router"):
            y, _ = w.moe(f)
            if mc.variant.upper() == "RESIDUAL_MOE":
                y = y + f
            return base + y
        gu = self._lin(f, li, "gate_up", w.gate_up, getattr(w, "gate_up_bias", None))
        act = F.glu_fwd(gu, mc.act_kernel) if mc.gated else F.act_fwd(gu, mc.act_kernel)
        return self._lin(act, li, "down", w.down, getattr(w, "down_bias", None), base)

    # ------------------------------------------------------------------ request management
    def add_request(self, tokens, max_tokens=64, sampling: Optional[SamplerConfig] = None, priority=0,
                    deadline=float("inf"), stop_ids=(), on_token=None) -> Request:
        r = Request(list(tokens), max_tokens, sampling or SamplerConfig(), next(self._ids), priority, deadline,
                    tuple(stop_ids), on_token)
        r.t_submit = time.perf_counter()
        heapq.heappush(self.waiting, (-priority, deadline, r.id, r))   # priority desc, deadline asc, FIFO
        return r

    def has_pending(self) -> bool:
        return bool(self.waiting or self.running or self._inflight is not None)

    def _release(self, r: Request):
        for p in r.pages:
            self.cache.allocator.release(p)
        r.pages = []

    # ------------------------------------------------------------------ model passes
    def _layers_prefill(self, ids, pos0, r: Request, all_positions: bool = False):
        """Prompt tokens ids[pos0:] of one sequence; K/V of all of them go to the pages.  Returns the
        hidden state of the last token (of every new token with ``all_positions``).  (Prefix pages already hold
        positions < pos0.)"""
        m, mc = self.model, self.model.cfg
        dev = self.device
        Hq, Hkv, D = mc.num_heads, mc.num_kv_heads, mc.head_dim
        S = len(ids) - pos0
        t = torch.tensor(ids[pos0:], dtype=torch.int64, device=dev)
        h = F.embedding_fwd(t, m.tok_embeddings.data, None, 0)
        if m.pos_embeddings is not None:
            h = h + m.pos_embeddings.data[pos0:pos0 + S]
        rope = m.rope(dev)
        positions = torch.arange(pos0, pos0 + S, dtype=torch.int32, device=dev)
        slots = torch.tensor([r.pages[p // PAGE] * PAGE + p % PAGE for p in range(pos0, pos0 + S)], dtype=torch.int64,
                             device=dev)
        pages_dev = None
        for li, w in enumerate(m.layers):
            a, _ = _norm_fwd(mc, h, w.attention_norm, getattr(w, "attention_norm_bias", None))
            qkv = self._lin(a, li, "qkv", w.qkv, getattr(w, "qkv_bias", None))
            if rope is not None:
                F.rope_(qkv, rope[0], rope[1], Hq + Hkv, D, S, positions=positions)
            self.cache.append(li, qkv, Hq * D, (Hq + Hkv) * D, slots)
            if pos0 == 0:
                o, _ = F.attn_fwd(qkv, qkv, qkv, 1, S, Hq, Hkv, D, k_col0=Hq * D, v_col0=(Hq + Hkv) * D)
            else:
                # suffix after a cached prefix: the prefix and the rows just appended come out of the pages as contiguous
                # bf16 rows (dequantised), and the new tokens run through the tensor-core attention kernel as the last S
                # positions of a pos0 + S long sequence
                if pages_dev is None:
                    pages_dev = torch.tensor(r.pages, dtype=torch.int32, device=dev)
                kk, vv = self.cache.gather(li, pages_dev, pos0 + S)
                o, _ = F.attn_fwd(qkv, kk, vv, 1, S, Hq, Hkv, D, kv_len=pos0 + S)
            if mc.use_parallel_residual:
                attn = self._lin(o, li, "o", w.o, getattr(w, "o_bias", None))
                f, _ = _norm_fwd(mc, h, w.ffn_norm, getattr(w, "ffn_norm_bias", None))
                base = h
            else:
                base = self._lin(o, li, "o", w.o, getattr(w, "o_bias", None), h)
                f, _ = _norm_fwd(mc, base, w.ffn_norm, getattr(w, "ffn_norm_bias", None))
            h = self._ffn(li, w, f, base)
            if mc.use_parallel_residual:
                h = h + attn
        return h if all_positions else h[-1:]

    def _layers_prefill_batch(self, reqs: List[Request]):
        """Whole prompts of several sequences in one pass: rows are [B, S_max] with the shorter prompts padded on the right
        (causal attention keeps padding from reaching real tokens; padded rows carry slot -1 and are not cached).
        Returns the hidden state of every sequence's last prompt token, [B, H]."""
        m, mc = self.model, self.model.cfg
        dev = self.device
        Hq, Hkv, D = mc.num_heads, mc.num_kv_heads, mc.head_dim
        B, S = len(reqs), max(len(r.tokens) for r in reqs)
        ids = torch.zeros((B, S), dtype=torch.int64)
        slots = torch.full((B, S), -1, dtype=torch.int64)
        for b, r in enumerate(reqs):
            n = len(r.tokens)
            ids[b, :n] = torch.tensor(r.tokens, dtype=torch.int64)
            pg = torch.tensor(r.pages, dtype=torch.int64)
            pos = torch.arange(n)
            slots[b, :n] = pg[pos // PAGE] * PAGE + pos % PAGE
        ids, slots = ids.to(dev).reshape(-1), slots.to(dev).reshape(-1)
        h = F.embedding_fwd(ids, m.tok_embeddings.data, None, 0)
        if m.pos_embeddings is not None:
            h = h + m.pos_embeddings.data[:S].repeat(B, 1)
        rope = m.rope(dev)
        positions = torch.arange(S, dtype=torch.int32, device=dev).repeat(B)
        for li, w in enumerate(m.layers):
            a, _ = _norm_fwd(mc, h, w.attention_norm, getattr(w, "attention_norm_bias", None))
            qkv = self._lin(a, li, "qkv", w.qkv, getattr(w, "qkv_bias", None))
            if rope is not None:
                F.rope_(qkv, rope[0], rope[1], Hq + Hkv, D, S, positions=positions)
            self.cache.append(li, qkv, Hq * D, (Hq + Hkv) * D, slots)
            o, _ = F.attn_fwd(qkv, qkv, qkv, B, S, Hq, Hkv, D, k_col0=Hq * D, v_col0=(Hq + Hkv) * D)
            if mc.use_parallel_residual:
                attn = self._lin(o, li, "o", w.o, getattr(w, "o_bias", None))
                f, _ = _norm_fwd(mc, h, w.ffn_norm, getattr(w, "ffn_norm_bias", None))
                base = h
            else:
                base = self._lin(o, li, "o", w.o, getattr(w, "o_bias", None), h)
                f, _ = _norm_fwd(mc, base, w.ffn_norm, getattr(w, "ffn_norm_bias", None))
            h = self._ffn(li, w, f, base)
            if mc.use_parallel_residual:
                h = h + attn
        last = torch.tensor([b * S + len(r.tokens) - 1 for b, r in enumerate(reqs)], dtype=torch.int64, device=dev)
        return h[last]

    def _prefill_fresh(self, fresh: List[Request], finished: list):
        """Groups the newly admitted prompts (sorted by length, so padding stays small) under the padded-token budget and
        prefills each group in one pass; then samples every sequence's first token."""
        fresh = sorted(fresh, key=lambda r: len(r.tokens))
        groups, cur = [], []
        for r in fresh:
            if cur and (len(cur) + 1) * len(r.tokens) > self.cfg.max_prefill_tokens:
                groups.append(cur)
                cur = []
            cur.append(r)
        if cur:
            groups.append(cur)
        for grp in groups:
            t0 = time.perf_counter()
            h = self._layers_prefill_batch(grp) if len(grp) > 1 else self._layers_prefill(grp[0].tokens, 0, grp[0])
            toks = self._sample(self._logits(h), grp)
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            self.stats.prefill_ms += (time.perf_counter() - t0) * 1e3
            for r, tok in zip(grp, toks):
                n = len(r.tokens)
                self.stats.prompt_tokens += n
                if self.prefix:
                    self.prefix.insert(r.tokens, r.pages)
                r.pos = n
                r.t_first = time.perf_counter()
                self._emit(r, tok, finished)
                if not r.finished:
                    self.running.append(r)

    def _layers_decode(self, tokens, positions, block_table, slots):
        m, mc = self.model, self.model.cfg
        Hq, Hkv, D = mc.num_heads, mc.num_kv_heads, mc.head_dim
        B = tokens.shape[0]
        h = F.embedding_fwd(tokens, m.tok_embeddings.data, None, 0)
        if m.pos_embeddings is not None:
            h = h + m.pos_embeddings.data[positions.long()]
        rope = m.rope(self.device)
        lens = (positions + 1).to(torch.int32)
        for li, w in enumerate(m.layers):
            a, _ = _norm_fwd(mc, h, w.attention_norm, getattr(w, "attention_norm_bias", None))
            qkv = self._lin(a, li, "qkv", w.qkv, getattr(w, "qkv_bias", None))
            if rope is not None:
                F.rope_(qkv, rope[0], rope[1], Hq + Hkv, D, 1, positions=positions)
            self.cache.append(li, qkv, Hq * D, (Hq + Hkv) * D, slots)
            o = self.cache.decode(li, qkv[:, :Hq * D], block_table, lens, Hq)
            if mc.use_parallel_residual:
                attn = self._lin(o, li, "o", w.o, getattr(w, "o_bias", None))
                f, _ = _norm_fwd(mc, h, w.ffn_norm, getattr(w, "ffn_norm_bias", None))
                base = h
            else:
                base = self._lin(o, li, "o", w.o, getattr(w, "o_bias", None), h)
                f, _ = _norm_fwd(mc, base, w.ffn_norm, getattr(w, "ffn_norm_bias", None))
            h = self._ffn(li, w, f, base)
            if mc.use_parallel_residual:
                h = h + attn
        return h

    def _logits(self, h):
        m = self.model
        f, _ = _norm_fwd(m.cfg, h, m.norm, m.norm_bias)
        return F.gemm(f, m.lm_head.data)

    def _sample_dev(self, logits, reqs):
        """Sampled token ids as a device tensor [len(reqs)] (no host synchronisation)."""
        dev = logits.device
        # the per-row sampling parameters only change when the set of rows does: keep them on the device between steps
        key = tuple(r.id for r in reqs)
        cached = self._sample_cache
        if cached is None or cached[0] != key:
            vals = torch.tensor([[r.sampling.temperature, r.sampling.top_p, r.sampling.repetition_penalty] for r in reqs],
                                dtype=torch.float32).t().contiguous().to(dev)
            k = torch.tensor([0 if (r.sampling.reference_rule and r.sampling.top_p < 1) else r.sampling.top_k for r in reqs],
                             dtype=torch.int32, device=dev)
            cached = self._sample_cache = (key, vals[0], k, vals[1], vals[2])
        _, t, k, p, rp = cached
        hist = None
        if any(r.sampling.repetition_penalty != 1.0 for r in reqs):
            n = max(len(r.tokens) + len(r.out) for r in reqs)
            hist = torch.full((len(reqs), n), -1, dtype=torch.int32)
            for i, r in enumerate(reqs):
                seq = r.tokens + r.out
                hist[i, :len(seq)] = torch.tensor(seq, dtype=torch.int32)
            hist = hist.to(dev)
        self._step += 1
        return sample(logits, t, k, p, rp, hist, self.cfg.seed, self._step)

    def _sample(self, logits, reqs):
        return self._sample_dev(logits, reqs).tolist()

    # ------------------------------------------------------------------ scheduling
    @torch.no_grad()
    def step(self) -> List[Request]:
        """Admit + prefill what fits, then one decode token for every running sequence.  Returns the
        requests that finished during this step."""
        finished: List[Request] = []
        alloc = self.cache.allocator
        # ---- admission / prefill ----
        fresh: List[Request] = []
        while self.waiting and len(self.running) + len(fresh) < self.cfg.max_batch:
            r = self.waiting[0][3]
            n = min(len(r.tokens), self.max_len - 1)
            r.tokens = r.tokens[:n]
            shared = self.prefix.lookup(r.tokens) if self.prefix else []
            need = (n + r.max_tokens + PAGE - 1) // PAGE - len(shared)
            if need > alloc.num_free:
                if self.prefix and self.prefix.table and not self.running:
                    for p in shared:
                        alloc.release(p)
                    self.prefix.evict_all()
                    continue
                for p in shared:
                    alloc.release(p)
                break
            heapq.heappop(self.waiting)
            r.pages = shared + [alloc.alloc() for _ in range((n + PAGE - 1) // PAGE - len(shared))]
            pos0 = len(shared) * PAGE
            if pos0 == 0 and self.cfg.batch_prefill:
                fresh.append(r)
                continue
            t0 = time.perf_counter()
            h = self._layers_prefill(r.tokens, pos0, r)
            tok = self._sample(self._logits(h), [r])[0]
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            self.stats.prefill_ms += (time.perf_counter() - t0) * 1e3
            self.stats.prompt_tokens += n
            self.stats.prefix_hit_tokens += pos0
            if self.prefix:
                self.prefix.insert(r.tokens, r.pages)
            r.pos = n
            r.t_first = time.perf_counter()
            self._emit(r, tok, finished)
            if not r.finished:
                self.running.append(r)
        if fresh:
            self._prefill_fresh(fresh, finished)
        # ---- one decode token for everything that is running ----
        # Pipelined form (CUDA, no repetition penalty): positions, slots and the block table are known on the host without
        # the previous step's tokens, and those tokens are on the device, so the next step is launched first and the
        # previous step's tokens are read (from a pinned buffer filled behind an event) while it runs.  End-of-sequence
        # tokens are therefore seen one step late: such a sequence runs one step too many, whose result is dropped (its
        # cache write lands in pages that are free or handed to a prefill enqueued later on the same stream).
        dev = self.device
        prev, self._inflight = self._inflight, None
        pipelined = (bool(self.cfg.pipeline_decode) and (dev.type == "cuda" or self.cfg.pipeline_decode == "force") and
                     all(r.sampling.repetition_penalty == 1.0 for r in self.running))
        if prev is not None and not pipelined:
            self._collect(prev, finished)
            prev = None
        def launch_set():
            pend_ = {id(r): i for i, r in enumerate(prev[0])} if prev is not None else {}
            # with its pending token counted, a sequence is decoded again only if that token does not end it by length
            return pend_, [r for r in self.running if id(r) not in pend_ or
                           (len(r.out) + 1 < r.max_tokens and len(r.tokens) + len(r.out) + 1 < self.max_len)]
        pend, reqs = launch_set()
        if prev is not None and reqs and self.cfg.cuda_graph and self._bucket(len(reqs)) not in self._graphs:
            # a graph for this batch size has to be captured first: do that with nothing in flight
            self._collect(prev, finished)
            prev = None
            pend, reqs = launch_set()
        if reqs:
            t0 = time.perf_counter()
            for r in reqs:
                if r.pos // PAGE >= len(r.pages):
                    r.pages.append(alloc.alloc())
            # host tokens (0 where the token is still on the device), positions, slots and the row of the previous step that
            # holds a pending token (-1: none) travel in one small upload; the block table only re-sends what changed
            packed = torch.tensor([[0 if id(r) in pend else r.out[-1] for r in reqs], [r.pos for r in reqs],
                                   [r.pages[r.pos // PAGE] * PAGE + r.pos % PAGE for r in reqs],
                                   [pend.get(id(r), -1) for r in reqs]], dtype=torch.int64).to(dev)
            tokens, positions, slots = packed[0], packed[1].to(torch.int32), packed[2]
            if pend:
                src = packed[3]
                tokens = torch.where(src >= 0, prev[1][src.clamp(min=0)], tokens)
            bt = self._block_table(reqs)
            if self.cfg.cuda_graph and dev.type == "cuda":
                bucket = self._bucket(len(reqs))
                g = self._graphs.get(bucket)
                if g is None:
                    g = self._graphs[bucket] = _DecodeGraph(self, bucket)
                logits = g.replay(tokens, positions, bt, slots)
            else:
                logits = self._logits(self._layers_decode(tokens, positions, bt, slots))
            for r in reqs:
                r.pos += 1
            toks_dev = self._sample_dev(logits, reqs)
            if pipelined:
                host = ev = None
                if dev.type == "cuda":
                    if self._tok_host is None:
                        self._tok_host = _pinned_token_buffers(dev, self.cfg.max_batch)
                    self._tok_flip = getattr(self, "_tok_flip", 0) ^ 1  # never the buffer the previous step is still read from
                    host = self._tok_host[self._tok_flip][:len(reqs)]
                    host.copy_(toks_dev, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record()
                self._inflight = (reqs, toks_dev, host, ev)
                if prev is not None:
                    self._collect(prev, finished)
            else:
                self._collect((reqs, toks_dev, None, None), finished)
            self.stats.decode_ms += (time.perf_counter() - t0) * 1e3
        elif prev is not None:
            self._collect(prev, finished)
        return finished

    @staticmethod
    def _bucket(n: int) -> int:
        b = 1
        while b < n:
            b *= 2
        return b

    def _collect(self, step, finished: list):
        """Read the tokens of a launched decode step and hand them to their requests (a request that has finished in the
        meantime - end of sequence seen one step late, or stopped from outside - drops its token)."""
        reqs, toks_dev, host, ev = step
        if host is not None:
            ev.synchronize()
            toks = host.tolist()
        else:
            toks = toks_dev.tolist()
        for r, tok in zip(reqs, toks):
            if not r.finished:
                self._emit(r, tok, finished)
        self.running = [r for r in self.running if not r.finished]

    def _block_table(self, reqs):
        """Device block table [len(reqs), max_pages] for the running sequences.  The table lives on the device; a step
        uploads only what changed since the last one - the page a sequence has just started, or the whole row when a
        different request now sits in that row - as one (index, value) list.  Entries past a sequence's last page may be
        stale: the kernels read pages below ceil(length / 16) only."""
        dev, mp = self.device, self.max_pages
        if self._bt_cache is None:
            self._bt_cache = (torch.zeros((self.cfg.max_batch, mp), dtype=torch.int32, device=dev), [])
        table, rows = self._bt_cache
        idx, val = [], []
        for i, r in enumerate(reqs):
            n = len(r.pages)
            have = rows[i] if i < len(rows) else None
            if have is None or have[0] != r.id or have[1] > n:
                lo = 0
            elif have[1] < n:
                lo = have[1]
            else:
                continue
            idx.extend(range(i * mp + lo, i * mp + n))
            val.extend(r.pages[lo:])
            if i < len(rows):
                rows[i] = (r.id, n)
            else:
                rows.append((r.id, n))
        del rows[len(reqs):]
        if idx:
            u = torch.tensor([idx, val], dtype=torch.int64).to(dev)
            table.view(-1).index_copy_(0, u[0], u[1].to(torch.int32))
        return table[:len(reqs)]

    def _emit(self, r: Request, tok: int, finished: list):
        r.out.append(tok)
        self.stats.generated_tokens += 1
        if r.on_token:
            r.on_token(tok)
        eos = self.tok.eos_id if self.tok is not None else -1
        if tok == eos or tok in r.stop_ids or len(r.out) >= r.max_tokens or len(r.tokens) + len(r.out) >= self.max_len:
            r.finished = True
            r.t_done = time.perf_counter()
            self._release(r)
            finished.append(r)

    # ------------------------------------------------------------------ convenience API
    def generate_batch(self, prompts: List[List[int]], max_tokens=64, sampling: Optional[SamplerConfig] = None):
        reqs = [self.add_request(p, max_tokens, sampling) for p in prompts]
        while self.has_pending():
            self.step()
        return [r.out for r in reqs]

    def generate(self, prompt: str, max_tokens=64, sampling: Optional[SamplerConfig] = None) -> str:
        ids = self.tok.encode(prompt)
        out = self.generate_batch([ids], max_tokens, sampling)[0]
        eos = self.tok.eos_id
        return self.tok.decode([t for t in out if t != eos])

    def generate_stream(self, prompt: str, on_text: Callable[[str], None], max_tokens=64,
                        sampling: Optional[SamplerConfig] = None):
        ids = self.tok.encode(prompt)
        acc: List[int] = []
        sent = [""]

        def on_tok(t):
            if t == self.tok.eos_id:
                return
            acc.append(t)
            text = self.tok.decode(acc)
            if not text.endswith("�"):       # hold back incomplete UTF-8 sequences
                on_text(text[len(sent[0]):])
                sent[0] = text
        r = self.add_request(ids, max_tokens, sampling, on_token=on_tok)
        while not r.finished:
            self.step()
        return r

    def generate_with_stats(self, prompt: str, max_tokens=64, sampling: Optional[SamplerConfig] = None):
        t0 = time.perf_counter()
        before = self.stats.generated_tokens
        text = self.generate(prompt, max_tokens, sampling)
        dt = time.perf_counter() - t0
        st = InferenceStats(**self.stats.__dict__)
        st.tokens_per_sec = (self.stats.generated_tokens - before) / max(dt, 1e-9)
        return text, st

    def reset_context(self):
        for r in self.running:
            self._release(r)
        self.running, self.waiting = [], []
        if self.prefix:
            self.prefix.evict_all()
