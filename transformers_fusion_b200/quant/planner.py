"""Bit-budget planning: which quantisation format each 256-weight block gets so that a tensor (or a
whole model) meets a target bits-per-weight.

* ``FormatRegistry`` - descriptors of the single formats, the two-tier and four-tier mixes, selection
  by target bpw or by measured error, and ``allocate_mix_blocks``: a greedy benefit-per-byte upgrade
  under a hard byte budget.
* ``FormatPlanner``  - importance scoring (|w|*|a| magnitude or a Fisher diagonal), ``allocate``,
  ``plan_for_model`` and ``plan_for_target``.

Reference counterparts: FormatPlanner (src/codec/format_planner.cpp:10-340), FormatRegistry
(src/codec/format_registry.cpp, include/quant/format_registry.h:68-160).  The byte accounting uses the
wire bits-per-weight of the block codec, so a plan's ``achieved_bpw`` is what the written file has."""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import codec

BASE_BITS = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32)


def _fmt(name):
    f = codec.parse_format(name)
    assert f >= 0, name
    return f


@dataclass
class FormatDescriptor:
    name: str
    id: int                 # wire format id
    bpw: float              # wire bits per weight
    grouped: bool = False
    lossless: bool = False
    description: str = ""


@dataclass
class MixDescriptor:
    name: str
    tiers: List[int]        # wire format ids, most precise first
    ratios: List[float]     # fraction of blocks per tier (sums to 1)
    effective_bpw: float = 0.0
    adaptive: bool = False

    @property
    def num_tiers(self):
        return len(self.tiers)


@dataclass
class WeightBlock:
    id: int
    weight_index: int
    num_weights: int
    assigned_format: int
    importance_score: float = 0.0


@dataclass
class FormatPlan:
    target_bpw: float = 0.0
    achieved_bpw: float = 0.0
    blocks: List[WeightBlock] = field(default_factory=list)
    uses_mix: bool = False
    selected_single: Optional[FormatDescriptor] = None
    selected_mix: Optional[MixDescriptor] = None

    def formats(self) -> np.ndarray:
        return np.array([b.assigned_format for b in self.blocks], dtype=np.uint8)

    def histogram(self):
        h = {}
        for b in self.blocks:
            n = codec.format_name(b.assigned_format)
            h[n] = h.get(n, 0) + 1
        return h


@dataclass
class QuantResult:
    """Blocks of one array encoded in one format."""
    format: int
    n: int
    block: int
    blocks: List[bytes]


class FormatRegistry:
    _singles = None
    _twi = None
    _four = None

    @classmethod
    def get_all_singles(cls) -> List[FormatDescriptor]:
        if cls._singles is None:
            out = []
            for b in BASE_BITS:
                f = _fmt(f"Q_{b}")
                out.append(FormatDescriptor(f"Q_{b}", f, codec.format_bpw(f), False, b == 32, f"{b}-bit per-block codec"))
            for b in BASE_BITS[:-1]:
                f = _fmt(f"Q_G_{b}")
                out.append(FormatDescriptor(f"Q_G_{b}", f, codec.format_bpw(f), True, False, f"{b}-bit grouped affine"))
            cls._singles = out
        return cls._singles

    @classmethod
    def get_all_twi_mixes(cls) -> List[MixDescriptor]:
        """Adjacent base formats blended 25/50/75 % (the half-step formats between two bit widths)."""
        if cls._twi is None:
            out = []
            base = [d for d in cls.get_all_singles() if not d.grouped]
            for lo, hi in zip(base[:-1], base[1:]):
                for r in (0.25, 0.5, 0.75):
                    bp = r * hi.bpw + (1 - r) * lo.bpw
                    out.append(MixDescriptor(f"MIX2_{hi.name}x{int(r * 100)}_{lo.name}", [hi.id, lo.id], [r, 1 - r], bp))
            cls._twi = out
        return cls._twi

    @classmethod
    def get_all_four_mixes(cls) -> List[MixDescriptor]:
        """Four consecutive base formats with a 10/20/30/40 % pyramid (few precise blocks, many cheap ones)."""
        if cls._four is None:
            out = []
            base = [d for d in cls.get_all_singles() if not d.grouped]
            ratios = [0.1, 0.2, 0.3, 0.4]
            for i in range(len(base) - 3):
                tiers = base[i:i + 4][::-1]
                bp = sum(r * t.bpw for r, t in zip(ratios, tiers))
                out.append(MixDescriptor("MIX4_" + "_".join(t.name for t in tiers), [t.id for t in tiers], list(ratios), bp, True))
            cls._four = out
        return cls._four

    @classmethod
    def get_single_format(cls, target_bpw: float) -> FormatDescriptor:
        """Most precise ungrouped single format that does not exceed the target (Q_1 when nothing fits)."""
        base = [d for d in cls.get_all_singles() if not d.grouped]
        fit = [d for d in base if d.bpw <= target_bpw + 1e-6]
        return max(fit, key=lambda d: d.bpw) if fit else base[0]

    @classmethod
    def _closest(cls, mixes, target):
        return min(mixes, key=lambda m: abs(m.effective_bpw - target))

    @classmethod
    def get_twi_mix(cls, target_bpw):
        return cls._closest(cls.get_all_twi_mixes(), target_bpw)

    @classmethod
    def get_four_mix(cls, target_bpw):
        return cls._closest(cls.get_all_four_mixes(), target_bpw)

    # ---- measured quality ----------------------------------------------------------------------
    @staticmethod
    def roundtrip(data: np.ndarray, fmt: int, block: int = 256) -> np.ndarray:
        data = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        out = np.empty_like(data)
        for o in range(0, data.size, block):
            seg = data[o:o + block]
            out[o:o + block] = codec.dequantize_block(fmt, codec.quantize_block(fmt, seg), seg.size)
        return out

    # ---- quantise / dequantise with a result record (reference: FormatRegistry::quantize ... actual_bpw,
    # include/quant/format_registry.h:121-147)
    @classmethod
    def quantize(cls, data, fmt, block: int = 256) -> "QuantResult":
        """Encode a flat array block by block into ``fmt`` (a descriptor, a format id or a name)."""
        f = fmt.id if isinstance(fmt, FormatDescriptor) else (_fmt(fmt) if isinstance(fmt, str) else int(fmt))
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        blocks = [codec.quantize_block(f, a[o:o + block]) for o in range(0, a.size, block)]
        return QuantResult(f, a.size, block, blocks)

    @classmethod
    def quantize_block(cls, block_data, fmt) -> "QuantResult":
        a = np.asarray(block_data, dtype=np.float32).reshape(-1)
        return cls.quantize(a, fmt, block=max(1, a.size))

    @staticmethod
    def dequantize(qr: "QuantResult", n: Optional[int] = None) -> np.ndarray:
        out = np.concatenate([codec.dequantize_block(qr.format, payload, min(qr.block, qr.n - i * qr.block))
                              for i, payload in enumerate(qr.blocks)]) if qr.blocks else np.zeros(0, np.float32)
        return out[: n or qr.n]

    @staticmethod
    def serialized_size_bytes(qr: "QuantResult") -> int:
        """Payload bytes plus the container's per-block framing (weight count, codebook size, index size: 12 bytes)."""
        return sum(len(b) for b in qr.blocks) + 12 * len(qr.blocks)

    @staticmethod
    def actual_bpw(qr: "QuantResult") -> float:
        return 8.0 * sum(len(b) for b in qr.blocks) / max(1, qr.n)

    @classmethod
    def quantize_q1(cls, data): return cls.quantize(data, "Q_1")

    @classmethod
    def quantize_q2(cls, data): return cls.quantize(data, "Q_2")

    @classmethod
    def quantize_q4(cls, data): return cls.quantize(data, "Q_4")

    @classmethod
    def quantize_q8(cls, data): return cls.quantize(data, "Q_8")

    @classmethod
    def quantize_q_twi_mix_1_5(cls, data, block_size: int = 256) -> List["QuantResult"]:
        """The 1.5-bit two-format mix: the half of the blocks with the larger energy in Q_2, the rest in Q_1; one result
        per block, in order."""
        a = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        spans = [a[o:o + block_size] for o in range(0, a.size, block_size)]
        energy = np.array([float((sp ** 2).mean()) for sp in spans])
        hi = set(np.argsort(-energy)[: len(spans) // 2].tolist())
        return [cls.quantize(sp, "Q_2" if i in hi else "Q_1", block_size) for i, sp in enumerate(spans)]

    @classmethod
    def quantize_q_sparse(cls, data, keep: float = 0.1) -> dict:
        """Sparse form: the largest ``keep`` fraction of the weights (by magnitude) as (index, fp16 value) pairs, the rest
        zero.  Returns {"n", "indices" int32, "values" float16}; ``dequantize_sparse`` restores the dense array."""
        a = np.asarray(data, dtype=np.float32).reshape(-1)
        k = max(1, int(round(keep * a.size)))
        idx = np.sort(np.argpartition(-np.abs(a), k - 1)[:k]).astype(np.int32)
        return {"n": a.size, "indices": idx, "values": a[idx].astype(np.float16)}

    @staticmethod
    def dequantize_sparse(sp: dict) -> np.ndarray:
        out = np.zeros(sp["n"], dtype=np.float32)
        out[sp["indices"]] = sp["values"].astype(np.float32)
        return out

    @classmethod
    def measure_mse(cls, a, b) -> float:
        a, b = np.asarray(a, dtype=np.float64).reshape(-1), np.asarray(b, dtype=np.float64).reshape(-1)
        return float(np.mean((a - b) ** 2))

    @classmethod
    def evaluate_format_quality(cls, data, fmt: FormatDescriptor, max_weights=1 << 16) -> float:
        d = np.asarray(data, dtype=np.float32).reshape(-1)[:max_weights]
        return cls.measure_mse(d, cls.roundtrip(d, fmt.id))

    @classmethod
    def evaluate_format_quality_weighted(cls, data, gradients, fmt: FormatDescriptor, fisher_weight=0.5, max_weights=1 << 16):
        d = np.asarray(data, dtype=np.float32).reshape(-1)[:max_weights]
        g = np.asarray(gradients, dtype=np.float32).reshape(-1)[:max_weights]
        e = (d - cls.roundtrip(d, fmt.id)).astype(np.float64) ** 2
        fw = g.astype(np.float64) ** 2
        fw = fw / max(fw.mean(), 1e-30)
        return float(np.mean(e * ((1 - fisher_weight) + fisher_weight * fw)))

    @classmethod
    def select_best_format(cls, target_bpw, data) -> FormatDescriptor:
        """Lowest measured error among the single formats (grouped ones included) within the budget."""
        fit = [d for d in cls.get_all_singles() if d.bpw <= target_bpw + 1e-6] or [cls.get_all_singles()[0]]
        top = sorted(fit, key=lambda d: -d.bpw)[:4]
        return min(top, key=lambda d: cls.evaluate_format_quality(data, d))

    @classmethod
    def select_best_mix(cls, target_bpw, data, block=256) -> MixDescriptor:
        cands = [m for m in cls.get_all_twi_mixes() + cls.get_all_four_mixes() if m.effective_bpw <= target_bpw + 1e-6]
        if not cands:
            return cls.get_twi_mix(target_bpw)
        cands = sorted(cands, key=lambda m: -m.effective_bpw)[:4]
        d = np.asarray(data, dtype=np.float32).reshape(-1)[:1 << 16]

        def err(m):
            fm = cls.allocate_mix_blocks(m, d, block)
            out = np.empty_like(d)
            for i, f in enumerate(fm):
                seg = d[i * block:(i + 1) * block]
                out[i * block:(i + 1) * block] = codec.dequantize_block(int(f), codec.quantize_block(int(f), seg), seg.size)
            return cls.measure_mse(d, out)
        return min(cands, key=err)

    @classmethod
    def allocate_mix_blocks(cls, mix: MixDescriptor, data, block: int = 256, importance=None) -> np.ndarray:
        """Per-block formats for ``data`` under the hard byte budget ceil(effective_bpw * n / 8).

        Every block starts in the cheapest tier; upgrades (one tier at a time) are taken greedily by
        estimated error reduction per extra byte until the budget is spent.  The error model is the
        uniform-quantiser one: block energy * 4^-bits, so high-energy (or high-importance) blocks are
        promoted first."""
        d = np.asarray(data, dtype=np.float32).reshape(-1)
        n = d.size
        nb = (n + block - 1) // block
        pad = np.zeros(nb * block, dtype=np.float32)
        pad[:n] = d
        energy = (pad.reshape(nb, block).astype(np.float64) ** 2).sum(1)
        if importance is not None:
            imp = np.asarray(importance, dtype=np.float64)[:nb]
            energy = energy * (imp / max(imp.mean(), 1e-30))
        lens = np.full(nb, block, dtype=np.int64)
        lens[-1] = n - (nb - 1) * block
        tiers = sorted(mix.tiers, key=lambda f: codec.format_bpw(f))          # cheap -> precise
        bpws = [codec.format_bpw(f) for f in tiers]
        cost = np.array([[codec.claimed_bytes(f, int(l)) for f in tiers] for l in np.unique(lens)])
        cost_of = {int(l): cost[i] for i, l in enumerate(np.unique(lens))}
        budget = int(np.ceil(mix.effective_bpw * n / 8.0))
        level = np.zeros(nb, dtype=np.int64)
        spent = sum(int(cost_of[int(l)][0]) for l in lens)

        def offer(b_, lv):
            extra = int(cost_of[int(lens[b_])][lv + 1] - cost_of[int(lens[b_])][lv])
            gain = energy[b_] * (4.0 ** (-bpws[lv]) - 4.0 ** (-bpws[lv + 1]))
            return (-gain / max(extra, 1), int(b_), lv, extra)
        heap = [offer(b_, 0) for b_ in range(nb)] if len(tiers) > 1 else []
        heapq.heapify(heap)
        while heap:
            _, b_, lv, extra = heapq.heappop(heap)
            if spent + extra > budget:
                continue                      # this block stays; cheaper upgrades of others may still fit
            level[b_] = lv + 1
            spent += extra
            if lv + 2 < len(tiers):
                heapq.heappush(heap, offer(b_, lv + 1))
        return np.array([tiers[l] for l in level], dtype=np.uint8)

    @classmethod
    def apply_forced_distribution(cls, target_bpw, num_formats, data=None):
        """``num_formats`` single formats around the target whose plain average stays within it."""
        base = [d for d in cls.get_all_singles() if not d.grouped]
        i = max(0, base.index(cls.get_single_format(target_bpw)))
        lo = max(0, i - num_formats // 2)
        sel = base[lo:lo + num_formats]
        while len(sel) > 1 and cls.compute_average_bpw(sel) > target_bpw + 1e-6:
            sel = sel[:-1] if lo == 0 else base[lo - 1:lo - 1 + len(sel)]
            lo = max(0, lo - 1)
        return sel

    @staticmethod
    def compute_average_bpw(assign: Sequence[FormatDescriptor]) -> float:
        return sum(d.bpw for d in assign) / max(1, len(assign))

    @classmethod
    def parse_format_name(cls, name: str) -> Optional[FormatDescriptor]:
        f = codec.parse_format(name)
        if f < 0:
            return None
        return FormatDescriptor(codec.format_name(f), f, codec.format_bpw(f), bool(codec.lib().tfb_format_is_grouped(f)),
                                f == codec.Q_32)

    @classmethod
    def get_format_table(cls) -> str:
        """Human-readable table of every wire format (the quant_format_list tool prints this)."""
        lines = [f"{'id':>4}  {'name':<16} {'bpw':>8}  {'bytes/256':>9}  {'kind':<10} wire-exact", "-" * 64]
        L = codec.lib()
        for f, _, _ in codec.all_formats():
            kind = "mix" if L.tfb_format_is_mix(f) else ("grouped" if L.tfb_format_is_grouped(f) else "plain")
            tier = ("", "K_L", "K_M", "K_H")[L.tfb_format_k_tier(f)]
            lines.append(f"{f:>4}  {codec.format_name(f):<16} {codec.format_bpw(f):>8.4f}  {codec.claimed_bytes(f, 256):>9}  "
                         f"{(kind + ' ' + tier).strip():<10} {'yes' if codec.is_wire_exact(f) else 'no'}")
        lines.append("")
        lines.append("two-tier mixes: " + ", ".join(f"{m.name}={m.effective_bpw:.3f}" for m in cls.get_all_twi_mixes()[:6]) + ", ...")
        lines.append("four-tier mixes: " + ", ".join(f"{m.name}={m.effective_bpw:.3f}" for m in cls.get_all_four_mixes()))
        return "\n".join(lines) + "\n"


class ImportanceMetric:
    MAGNITUDE = "magnitude"
    FISHER_DIAG = "fisher_diag"


class FormatPlanner:
    def __init__(self, target_bpw: float = 1.5):
        self.target_bpw = float(target_bpw)
        self._scores: Optional[np.ndarray] = None

    def set_target_bpw(self, b):
        self.target_bpw = float(b)

    def importance_scores(self):
        return self._scores

    @staticmethod
    def _blocks(t: torch.Tensor, block):
        f = t.detach().float().reshape(-1)
        nb = (f.numel() + block - 1) // block
        pad = torch.zeros(nb * block, dtype=torch.float32, device=f.device)
        pad[: f.numel()] = f
        cnt = torch.full((nb,), float(block), device=f.device)
        cnt[-1] = f.numel() - (nb - 1) * block
        return pad.view(nb, block), cnt

    def score_importance(self, weights, calibration_activations=None, block_size=256, metric=ImportanceMetric.MAGNITUDE):
        """MAGNITUDE: mean |w| * |a| per block (a = 1 without calibration data); FISHER_DIAG: see below."""
        if metric == ImportanceMetric.FISHER_DIAG:
            return self.score_importance_fisher(weights, calibration_activations, block_size)
        w, cnt = self._blocks(weights, block_size)
        if calibration_activations is not None:
            a, _ = self._blocks(calibration_activations, block_size)
            s = (w.abs() * a.abs()).sum(1) / cnt
        else:
            s = w.abs().sum(1) / cnt
        self._scores = s.cpu().numpy()
        return self._scores

    def score_importance_fisher(self, weights, gradients, block_size=256):
        """RMS gradient of the block times its RMS weight: the expected loss change of a relative
        perturbation (the reference scales by the block's first weight, format_planner.cpp:58)."""
        w, cnt = self._blocks(weights, block_size)
        g, _ = self._blocks(gradients, block_size)
        s = torch.sqrt((g * g).sum(1) / cnt) * torch.sqrt((w * w).sum(1) / cnt)
        self._scores = s.cpu().numpy()
        return self._scores

    @staticmethod
    def compute_format_mix(num_blocks: int, target_bpw: float):
        """{bits: block count} using the two base widths that bracket the target (nominal bits)."""
        bits = BASE_BITS
        if target_bpw >= 32:
            return {32: num_blocks}
        if target_bpw <= 1:
            return {1: num_blocks}
        up = next(i for i, b in enumerate(bits) if b >= target_bpw)
        if bits[up] == target_bpw:
            return {bits[up]: num_blocks}
        lo = up - 1
        r_up = (target_bpw - bits[lo]) / (bits[up] - bits[lo])
        n_up = int(np.floor(r_up * num_blocks))
        return {bits[up]: n_up, bits[lo]: num_blocks - n_up}

    def allocate(self, num_weight_blocks: int, weights_per_block: int = 256, last_block: Optional[int] = None) -> FormatPlan:
        """Assign formats so that the plan's wire bytes stay within target_bpw; the most important blocks
        (or, without scores, the first ones) get the precise tier."""
        plan = FormatPlan(target_bpw=self.target_bpw)
        t = self.target_bpw
        single = FormatRegistry.get_single_format(t)
        plan.selected_single = single
        base = [d for d in FormatRegistry.get_all_singles() if not d.grouped]
        i = base.index(single)
        nb = num_weight_blocks
        lens = np.full(nb, weights_per_block, dtype=np.int64)
        if last_block:
            lens[-1] = last_block
        total_w = int(lens.sum())
        budget = int(np.floor(t * total_w / 8.0))
        order = np.arange(nb) if self._scores is None else np.argsort(-self._scores[:nb], kind="stable")
        fm = np.full(nb, single.id, dtype=np.uint8)
        spent = sum(codec.claimed_bytes(single.id, int(l)) for l in lens)
        if i + 1 < len(base) and single.bpw < t - 1e-6 and spent <= budget:
            hi = base[i + 1]
            plan.uses_mix = True
            for b in order:
                extra = codec.claimed_bytes(hi.id, int(lens[b])) - codec.claimed_bytes(single.id, int(lens[b]))
                if spent + extra > budget:
                    break
                fm[b] = hi.id
                spent += extra
            r = float((fm == hi.id).mean())
            plan.selected_mix = MixDescriptor(f"MIX2_{hi.name}_{single.name}", [hi.id, single.id], [r, 1 - r],
                                              r * hi.bpw + (1 - r) * single.bpw)
        off = 0
        for b in range(nb):
            plan.blocks.append(WeightBlock(b, off, int(lens[b]), int(fm[b]),
                                           float(self._scores[b]) if self._scores is not None and b < len(self._scores) else 0.0))
            off += int(lens[b])
        plan.achieved_bpw = self.estimate_bpw(plan)
        return plan

    def plan_for_model(self, num_weights: int, block: int = 256) -> FormatPlan:
        nb = (num_weights + block - 1) // block
        return self.allocate(nb, block, num_weights - (nb - 1) * block)

    @staticmethod
    def plan_for_target(target_bpw: float, num_blocks: int, weights_per_block: int = 256) -> FormatPlan:
        return FormatPlanner(target_bpw).allocate(num_blocks, weights_per_block)

    @staticmethod
    def estimate_bpw(plan: FormatPlan) -> float:
        by = sum(codec.claimed_bytes(b.assigned_format, b.num_weights) for b in plan.blocks)
        return 8.0 * by / max(1, sum(b.num_weights for b in plan.blocks))
