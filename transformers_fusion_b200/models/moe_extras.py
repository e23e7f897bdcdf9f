"""Mixture-of-experts utilities beyond the core model: dense-to-MoE conversion, alternative routers, expert merging, a
dynamic expert pool, expert dropout and a disk / host / device expert prefetcher.

Reference counterparts: DenseToMoEPruner, SwitchV2Router, ExpertChoiceV2, ExpertMerger, DynamicExpertPool, ExpertDropout
(src/model/moe_enhance.cpp), ExpertPrefetcher (src/model/expert_prefetch.cpp, include/quant/expert_prefetch.h:73-105)."""
from __future__ import annotations

import os
import queue
import threading
import time
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch


class DenseToMoEPruner:
    """Splits a dense gated FFN (gate_up [2F, H], down [H, F]) into E experts by clustering its hidden units: units are
    grouped by the similarity of their input weights (k-means on the normalised ``up`` rows), each expert gets one group
    (padded / trimmed to F / E units), and the router is initialised to the group centroids so that tokens go to the expert
    whose units they excite most.  With top_k = E the mixture reproduces the dense layer exactly."""

    def __init__(self, num_experts: int, iters: int = 10, seed: int = 0):
        self.E, self.iters, self.seed = num_experts, iters, seed

    def convert(self, gate_up: torch.Tensor, down: torch.Tensor):
        F2, H = gate_up.shape
        F = F2 // 2
        assert F % self.E == 0
        per = F // self.E
        gate, up = gate_up[:F].float(), gate_up[F:].float()
        feat = torch.nn.functional.normalize(up, dim=1)
        g = torch.Generator().manual_seed(self.seed)
        cent = feat[torch.randperm(F, generator=g)[: self.E]].clone()
        for _ in range(self.iters):
            assign = self._balanced_assign(feat @ cent.t(), per)
            for e in range(self.E):
                cent[e] = torch.nn.functional.normalize(feat[assign == e].mean(0), dim=0)
        assign = self._balanced_assign(feat @ cent.t(), per)
        gu = torch.empty((self.E, 2 * per, H), dtype=gate_up.dtype)
        dn = torch.empty((self.E, H, per), dtype=down.dtype)
        for e in range(self.E):
            idx = (assign == e).nonzero().reshape(-1)
            gu[e, :per], gu[e, per:] = gate[idx].to(gate_up.dtype), up[idx].to(gate_up.dtype)
            dn[e] = down[:, idx]
        return gu, dn, cent.to(gate_up.dtype), assign

    def prune_ffn(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor):
        """The reference's call shape (include/quant/moe_enhance.h: DenseToMoEPruner::prune_ffn): separate gate [F, H] and
        up [F, H] matrices and down [H, F] of a dense FFN -> (expert gate_up, expert down, router initialisation)."""
        return self.convert(torch.cat([gate, up], 0), down)

    @staticmethod
    def _balanced_assign(score: torch.Tensor, per: int) -> torch.Tensor:
        """Greedy capacity-constrained assignment: most confident units choose first."""
        F, E = score.shape
        order = torch.argsort(score.max(1).values, descending=True)
        cap = [per] * E
        out = torch.empty(F, dtype=torch.long)
        for u in order.tolist():
            for e in torch.argsort(score[u], descending=True).tolist():
                if cap[e] > 0:
                    out[u], cap[e] = e, cap[e] - 1
                    break
        return out


class SwitchV2Router:
    """Top-1 routing with multiplicative jitter during training, a capacity limit per expert and a router z-loss."""

    def __init__(self, num_experts, capacity_factor=1.25, jitter=0.01, z_weight=1e-3):
        self.E, self.cf, self.jitter, self.zw = num_experts, capacity_factor, jitter, z_weight

    def route(self, logits: torch.Tensor, training=False, generator=None):
        T = logits.shape[0]
        lf = logits.float()
        if training and self.jitter > 0:
            lf = lf * (1 + (torch.rand(lf.shape, generator=generator) * 2 - 1).to(lf.device) * self.jitter)
        p = torch.softmax(lf, -1)
        w, idx = p.max(-1)
        cap = int(self.cf * T / self.E + 0.999)
        pos = torch.zeros(T, dtype=torch.long, device=lf.device)
        for e in range(self.E):
            m = idx == e
            pos[m] = torch.arange(int(m.sum()), device=lf.device)
        kept = pos < cap
        f = torch.bincount(idx, minlength=self.E).float() / T
        aux = self.E * (f * p.mean(0)).sum() + self.zw * (torch.logsumexp(lf, -1) ** 2).mean()
        return idx, w * kept, kept, aux


    def forward(self, logits: torch.Tensor, tokens: Optional[int] = None) -> torch.Tensor:
        """Dispatch matrix [T, E]: the routing weight where a token was kept by its expert, 0 elsewhere (evaluation mode)."""
        idx, w, kept, _ = self.route(logits, training=False)
        out = torch.zeros(logits.shape, dtype=torch.float32, device=logits.device)
        out[torch.arange(logits.shape[0], device=logits.device), idx] = w
        return out


class ExpertChoiceV2:
    """Experts pick tokens: every expert takes its ``capacity`` highest-scoring tokens, so the load is perfectly balanced;
    a token may be served by several experts or by none."""

    def __init__(self, num_experts, capacity_factor=2.0):
        self.E, self.cf = num_experts, capacity_factor

    def route(self, logits: torch.Tensor):
        T = logits.shape[0]
        cap = max(1, int(self.cf * T / self.E))
        p = torch.softmax(logits.float(), -1)            # over experts, per token
        w, tok = p.t().topk(min(cap, T), dim=1)          # [E, cap]
        return tok, w

    def combine(self, x, tok, w, expert_fn):
        y = torch.zeros_like(x, dtype=torch.float32)
        for e in range(self.E):
            y.index_add_(0, tok[e], expert_fn(e, x[tok[e]]).float() * w[e][:, None])
        return y.to(x.dtype)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, expert_fn=None) -> torch.Tensor:
        """Route and combine in one call; without ``expert_fn`` every expert is the identity (the weighted tokens come
        back, which shows who was served and how strongly)."""
        tok, w = self.route(logits)
        return self.combine(x, tok, w, expert_fn or (lambda e, rows: rows))


class ExpertMerger:
    """Merges the most similar experts (cosine similarity of their flattened weights), usage-weighted, until ``target``
    experts remain; returns the merged weights and the old -> new expert map."""

    @staticmethod
    def merge(gate_up: torch.Tensor, down: torch.Tensor, target: int, usage: Optional[torch.Tensor] = None):
        E = gate_up.shape[0]
        usage = (usage.float() if usage is not None else torch.ones(E)).clone()
        gu, dn = [gate_up[e].float().clone() for e in range(E)], [down[e].float().clone() for e in range(E)]
        groups = [[e] for e in range(E)]
        while len(gu) > target:
            flat = torch.stack([torch.nn.functional.normalize(torch.cat([a.reshape(-1), b.reshape(-1)]), dim=0) for a, b in zip(gu, dn)])
            sim = flat @ flat.t()
            sim.fill_diagonal_(-2)
            i, j = divmod(int(sim.argmax()), sim.shape[0])
            i, j = min(i, j), max(i, j)
            wi, wj = usage[i], usage[j]
            gu[i] = (gu[i] * wi + gu[j] * wj) / (wi + wj)
            dn[i] = (dn[i] * wi + dn[j] * wj) / (wi + wj)
            usage[i] = wi + wj
            groups[i] += groups[j]
            del gu[j], dn[j], groups[j]
            usage = torch.cat([usage[:j], usage[j + 1:]])
        mapping = {old: new for new, g in enumerate(groups) for old in g}
        return torch.stack(gu).to(gate_up.dtype), torch.stack(dn).to(down.dtype), mapping


class DynamicExpertPool:
    """Grows and shrinks the expert set from running utilisation: an expert whose share of tokens exceeds ``split_above`` is
    duplicated (with noise), one whose share stays under ``drop_below`` is removed."""

    def __init__(self, gate_up, down, router, split_above=0.5, drop_below=0.01, min_experts=2, max_experts=64, momentum=0.9):
        self.gu, self.dn, self.router = gate_up.clone(), down.clone(), router.clone()
        self.split, self.drop, self.min, self.max, self.mom = split_above, drop_below, min_experts, max_experts, momentum
        self.share = torch.full((gate_up.shape[0],), 1.0 / gate_up.shape[0])

    @property
    def num_experts(self):
        return self.gu.shape[0]

    def count(self) -> int:
        return self.num_experts

    def add_expert(self, gate_up: torch.Tensor, down: Optional[torch.Tensor] = None, router_row: Optional[torch.Tensor] = None) -> int:
        """Append an expert (its router row defaults to the mean of the existing rows); returns its index, or -1 when the
        pool is full."""
        if self.num_experts >= self.max:
            return -1
        down = down if down is not None else self.dn.float().mean(0).to(self.dn.dtype)
        row = router_row if router_row is not None else self.router.float().mean(0).to(self.router.dtype)
        self.gu = torch.cat([self.gu, gate_up.reshape(1, *self.gu.shape[1:]).to(self.gu.dtype)])
        self.dn = torch.cat([self.dn, down.reshape(1, *self.dn.shape[1:]).to(self.dn.dtype)])
        self.router = torch.cat([self.router, row.reshape(1, -1)])
        new_share = 1.0 / (self.num_experts)
        self.share = torch.cat([self.share * (1 - new_share), torch.tensor([new_share])])
        return self.num_experts - 1

    def remove_expert(self, idx: int) -> bool:
        if not 0 <= idx < self.num_experts or self.num_experts <= self.min:
            return False
        keep = [i for i in range(self.num_experts) if i != idx]
        self.gu, self.dn, self.router, self.share = self.gu[keep], self.dn[keep], self.router[keep], self.share[keep]
        self.share = self.share / self.share.sum().clamp(min=1e-12)
        return True

    def observe(self, expert_indices):
        c = torch.bincount(expert_indices.reshape(-1).cpu(), minlength=self.num_experts).float()
        self.share = self.mom * self.share + (1 - self.mom) * c / c.sum().clamp(min=1)

    def adapt(self, generator=None) -> Dict[str, List[int]]:
        log = {"split": [], "dropped": []}
        hot = [e for e in range(self.num_experts) if self.share[e] > self.split]
        for e in hot:
            if self.num_experts >= self.max:
                break
            n = lambda t: t + 0.01 * t.float().std().item() * torch.randn(t.shape, generator=generator).to(t.dtype)
            self.gu = torch.cat([self.gu, n(self.gu[e:e + 1])])
            self.dn = torch.cat([self.dn, n(self.dn[e:e + 1])])
            self.router = torch.cat([self.router, n(self.router[e:e + 1])])
            half = self.share[e] / 2
            self.share[e] = half
            self.share = torch.cat([self.share, half.reshape(1)])
            log["split"].append(e)
        cold = [e for e in range(self.num_experts) if self.share[e] < self.drop]
        for e in sorted(cold, reverse=True):
            if self.num_experts <= self.min:
                break
            keep = [i for i in range(self.num_experts) if i != e]
            self.gu, self.dn, self.router, self.share = self.gu[keep], self.dn[keep], self.router[keep], self.share[keep]
            log["dropped"].append(e)
        self.share = self.share / self.share.sum()
        return log


class ExpertDropout:
    """During training whole experts are masked out of the routing (their logits set to -inf) with probability ``p``; at
    least ``keep_min`` experts always survive."""

    def __init__(self, p=0.1, keep_min=2):
        self.p, self.keep_min = p, keep_min

    def get_active_count(self, total: int) -> int:
        """Experts expected to stay active out of ``total`` (never fewer than ``keep_min``)."""
        return max(min(self.keep_min, total), int(round(total * (1.0 - self.p))))

    def get_mask(self, total: int, generator=None) -> List[bool]:
        """One draw of the keep-mask over ``total`` experts (True = active)."""
        drop = torch.rand(total, generator=generator) < self.p
        if int((~drop).sum()) < min(self.keep_min, total):
            drop[torch.randperm(total, generator=generator)[: self.keep_min]] = False
        return (~drop).tolist()

    def __call__(self, logits: torch.Tensor, training=True, generator=None):
        if not training or self.p <= 0:
            return logits
        E = logits.shape[-1]
        drop = torch.rand(E, generator=generator) < self.p
        if int((~drop).sum()) < self.keep_min:
            drop[torch.randperm(E, generator=generator)[: self.keep_min]] = False
        return logits.masked_fill(drop.to(logits.device), float("-inf"))


class ExpertPrefetcher:
    """Three tiers for expert weights: disk (one file per expert) -> pinned host cache -> device cache, both LRU.  A worker
    thread serves prefetch requests (the router's prediction for the next layer); ``get`` blocks (bounded) until the expert
    is on the device."""

    def __init__(self, directory: str, device="cpu", host_slots=8, device_slots=2):
        self.dir, self.device = directory, torch.device(device)
        os.makedirs(directory, exist_ok=True)
        self.host: "OrderedDict[int, Dict[str, torch.Tensor]]" = OrderedDict()
        self.dev: "OrderedDict[int, Dict[str, torch.Tensor]]" = OrderedDict()
        self.host_slots, self.device_slots = host_slots, device_slots
        self.cv = threading.Condition()
        self.q: "queue.Queue" = queue.Queue()
        self.stats = {"disk_loads": 0, "host_hits": 0, "device_hits": 0}
        self.worker = threading.Thread(target=self._work, daemon=True)
        self.worker.start()

    def _path(self, e):
        return os.path.join(self.dir, f"expert_{e}.pt")

    def store(self, e: int, tensors: Dict[str, torch.Tensor]):
        torch.save({k: v.detach().cpu() for k, v in tensors.items()}, self._path(e))

    def _to_host(self, e):
        if e in self.host:
            self.host.move_to_end(e)
            self.stats["host_hits"] += 1
            return self.host[e]
        t = torch.load(self._path(e), map_location="cpu", weights_only=True)
        if self.device.type == "cuda":
            t = {k: v.pin_memory() for k, v in t.items()}
        self.stats["disk_loads"] += 1
        self.host[e] = t
        while len(self.host) > self.host_slots:
            self.host.popitem(last=False)
        return t

    def _to_device(self, e):
        with self.cv:
            if e in self.dev:
                self.dev.move_to_end(e)
                return
        h = self._to_host(e)
        d = {k: v.to(self.device, non_blocking=True) for k, v in h.items()}
        with self.cv:
            self.dev[e] = d
            while len(self.dev) > self.device_slots:
                self.dev.popitem(last=False)
            self.cv.notify_all()

    def _work(self):
        while True:
            e = self.q.get()
            if e is None:
                return
            try:
                self._to_device(e)
            except Exception:
                with self.cv:
                    self.cv.notify_all()

    def prefetch(self, experts):
        for e in experts:
            self.q.put(int(e))

    # ---- per-layer form of the reference (include/quant/expert_prefetch.h:73-105): experts are addressed by (layer, expert)
    def initialize(self, num_experts: int = 0, num_layers: int = 1):
        self.num_experts_per_layer, self.num_layers = int(num_experts), int(num_layers)
        self.wait_ms_total, self.waits, self.misses, self.evictions = 0.0, 0, 0, 0
        return self

    def _key(self, layer_id: int, expert_id: int) -> int:
        return int(layer_id) * max(1, getattr(self, "num_experts_per_layer", 0) or 1 << 16) + int(expert_id)

    def set_expert_source(self, layer_id: int, expert_id: int, tensors):
        """Register where an expert's weights come from: a dict of tensors (or one packed tensor), written to the disk tier."""
        self.store(self._key(layer_id, expert_id), tensors if isinstance(tensors, dict) else {"packed": tensors})

    def set_expert_segments(self, layer_id: int, expert_id: int, segments):
        """Several separately stored pieces (gate, up, down) of one expert: a list of tensors or (name, tensor) pairs."""
        named = {(s[0] if isinstance(s, tuple) else f"segment{i}"): (s[1] if isinstance(s, tuple) else s) for i, s in enumerate(segments)}
        self.store(self._key(layer_id, expert_id), named)

    def schedule_prefetch(self, layer_id: int, expert_ids):
        self.prefetch(self._key(layer_id, e) for e in expert_ids)

    def get_expert_weights(self, layer_id: int, expert_id: int, timeout_s: float = 5.0):
        k = self._key(layer_id, expert_id)
        with self.cv:
            hit = k in self.dev
        t0 = time.perf_counter()
        out = self.get(k, timeout_s)
        if not hit and hasattr(self, "waits"):
            self.misses += 1
            self.waits += 1
            self.wait_ms_total += (time.perf_counter() - t0) * 1e3
        return out

    def release_expert(self, layer_id: int, expert_id: int):
        """Drop an expert from the device tier (it stays in the host tier until that fills up)."""
        with self.cv:
            if self.dev.pop(self._key(layer_id, expert_id), None) is not None and hasattr(self, "evictions"):
                self.evictions += 1

    def get_stats(self) -> Dict[str, float]:
        return {"prefetch_hits": self.stats["device_hits"], "prefetch_misses": getattr(self, "misses", 0),
                "evictions": getattr(self, "evictions", 0), "disk_loads": self.stats["disk_loads"],
                "avg_wait_ms": getattr(self, "wait_ms_total", 0.0) / max(1, getattr(self, "waits", 0))}

    def get(self, e: int, timeout_s=5.0) -> Dict[str, torch.Tensor]:
        with self.cv:
            if e in self.dev:
                self.dev.move_to_end(e)
                self.stats["device_hits"] += 1
                return self.dev[e]
        self.q.put(int(e))
        end = time.time() + timeout_s
        with self.cv:
            while e not in self.dev:
                rest = end - time.time()
                if rest <= 0:
                    raise TimeoutError(f"expert {e} was not loaded in time")
                self.cv.wait(rest)
            return self.dev[e]

    def close(self):
        self.q.put(None)
        self.worker.join(timeout=2)
