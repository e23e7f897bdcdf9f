"""Host-side parallel planners.  They work on plain tensors / lists and double as CPU oracles for the device
collectives and the fused tensor-parallel kernels.

Reference counterpart: engines/trainer/dense/parallel.h:13-56, parallel.cpp:1-196."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence

import torch


@dataclass
class RankSlice:
    rank: int = 0
    world: int = 1
    start: int = 0
    count: int = 0


def slice_for(n: int, rank: int, world: int) -> RankSlice:
    """Contiguous split of n items; the first n % world ranks hold one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank / world")
    base, rem = divmod(n, world)
    return RankSlice(rank, world, rank * base + min(rank, rem), base + (1 if rank < rem else 0))


def ring_allreduce_sum(bufs: List[torch.Tensor]) -> None:
    """In-place ring all-reduce (reduce-scatter then all-gather, W - 1 steps each) over one buffer per rank."""
    W = len(bufs)
    if W <= 1:
        return
    n = bufs[0].numel()
    if any(b.numel() != n for b in bufs):
        raise ValueError("buffers differ in size")
    sl = [slice_for(n, c, W) for c in range(W)]
    seg = lambda c: slice(sl[c % W].start, sl[c % W].start + sl[c % W].count)
    flat = [b.view(-1) for b in bufs]
    for step in range(W - 1):                         # reduce-scatter: rank r sends chunk r - step to r + 1
        sends = [flat[r][seg(r - step)].clone() for r in range(W)]
        for r in range(W):
            flat[(r + 1) % W][seg(r - step)] += sends[r]
    for step in range(W - 1):                         # all-gather: rank r forwards its finished chunk r + 1 - step
        sends = [flat[r][seg(r + 1 - step)].clone() for r in range(W)]
        for r in range(W):
            flat[(r + 1) % W][seg(r + 1 - step)] = sends[r]


def broadcast_bufs(bufs: List[torch.Tensor], src: int = 0) -> None:
    for r, b in enumerate(bufs):
        if r != src:
            b.copy_(bufs[src])


def average_grad_slices(grads: List[torch.Tensor], world: int) -> None:
    for g in grads:
        g.div_(world)


@dataclass
class TPSplit:
    shards: List[torch.Tensor]
    dim: int = 0


def tp_split_cols(w: torch.Tensor, world: int) -> TPSplit:
    """Column-parallel split of W [out, in] along ``out`` (each rank computes a slice of the output features)."""
    if w.shape[0] % world:
        raise ValueError("output features do not divide by the TP degree")
    return TPSplit([s.contiguous() for s in w.chunk(world, 0)], 0)


def tp_gather_cols(shards: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat(list(shards), 0)


def tp_split_rows(w: torch.Tensor, world: int) -> TPSplit:
    """Row-parallel split along ``in`` (each rank consumes a slice of the input features; outputs are summed)."""
    if w.shape[1] % world:
        raise ValueError("input features do not divide by the TP degree")
    return TPSplit([s.contiguous() for s in w.chunk(world, 1)], 1)


def tp_gather_rows(shards: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat(list(shards), 1)


@dataclass
class ShardPlan:
    entries: List[tuple] = field(default_factory=list)       # (name, rank, bytes)
    rank_bytes: List[int] = field(default_factory=list)
    total_bytes: int = 0

    def imbalance(self) -> float:
        """max rank load / mean rank load - 1 (0 = perfectly even)."""
        if not self.rank_bytes or self.total_bytes <= 0:
            return 0.0
        return max(self.rank_bytes) / (self.total_bytes / len(self.rank_bytes)) - 1.0


def plan_shards(names: Sequence[str], numels: Sequence[int], world: int, bytes_per_el: int = 4) -> ShardPlan:
    """Whole-tensor placement: each tensor, in the given order, goes to the currently lightest rank."""
    if len(names) != len(numels):
        raise ValueError("names / sizes mismatch")
    if world <= 0:
        raise ValueError("bad world")
    p = ShardPlan(rank_bytes=[0] * world)
    for name, n in zip(names, numels):
        r = min(range(world), key=lambda q: p.rank_bytes[q])
        b = int(n) * bytes_per_el
        p.entries.append((name, r, b))
        p.rank_bytes[r] += b
        p.total_bytes += b
    return p


@dataclass
class PipePlan:
    layer_stage: List[int]
    stage_layers: List[int]
    stages: int = 1


def plan_pipeline(layers: int, stages: int) -> PipePlan:
    if stages <= 0 or layers <= 0:
        raise ValueError("bad pipeline plan")
    ls = [min(stages - 1, l * stages // layers) for l in range(layers)]
    return PipePlan(ls, [ls.count(s) for s in range(stages)], stages)
