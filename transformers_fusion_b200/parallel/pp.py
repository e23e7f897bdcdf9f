"""Pipeline parallelism: the layer stack is cut into contiguous stages (stage 0 owns the embedding, the last stage
the final norm, LM head and loss); micro-batches flow through the stages as point-to-point sends of the hidden state
[mb * S, H] and of its gradient.  Schedules: GPipe (all forwards, then all backwards) and 1F1B (warm-up forwards,
steady one-forward-one-backward, cool-down backwards), which bounds the live activations of a stage by the number of
stages after it instead of the number of micro-batches.  Transport is ``torch.distributed`` send / recv (NCCL between
GPUs, gloo on CPU); each stage runs the hand-written block forward / backward of the dense model.

``DualPipe`` keeps the reference's bookkeeping-only skeleton (bidirectional slot table, no execution).

Reference counterparts: PipelineParallel (include/quant/pipeline.h:22-120, src/trainer/pipeline.cpp: split_model :47-110,
GPipe :150-240, 1F1B :250-420, send/recv via ctx.broadcast :301-341), DualPipe :430-488."""
from __future__ import annotations

import time
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..models.dense import block_backward, block_forward
from ..ops import functional as F
from .collectives import DistributedContext


def split_model(num_layers: int, num_stages: int, balance_weights: Optional[Sequence[float]] = None):
    """[(lo, hi)] layer range per stage.  Default: ceil(num_layers / num_stages) layers per stage (the last stages may
    get fewer); with ``balance_weights`` (relative cost per stage) ranges are proportional to the weights."""
    if balance_weights:
        tot = float(sum(balance_weights))
        cuts, acc = [0], 0.0
        for w in balance_weights[:-1]:
            acc += w
            cuts.append(min(num_layers, max(cuts[-1], round(num_layers * acc / tot))))
        cuts.append(num_layers)
        return [(cuts[i], cuts[i + 1]) for i in range(num_stages)]
    per = -(-num_layers // num_stages)
    return [(min(num_layers, s * per), min(num_layers, (s + 1) * per)) for s in range(num_stages)]


class PipelineParallel:
    def __init__(self, model, num_stages: int, stage_id: int, ctx: Optional[DistributedContext] = None,
                 num_microbatches: int = 4, balance_weights=None, stage_ranks: Optional[Sequence[int]] = None):
        self.model, self.S, self.sid = model, num_stages, stage_id
        # global rank of every stage of this pipeline (identity unless the pipeline is one slice of a larger job)
        self.stage_ranks = list(stage_ranks) if stage_ranks is not None else list(range(num_stages))
        self.ctx = ctx or DistributedContext(stage_id, num_stages)
        self.num_microbatches = num_microbatches
        self.balance = balance_weights
        self.lo, self.hi = split_model(model.cfg.num_layers, num_stages, balance_weights)[stage_id]
        self.first, self.last = stage_id == 0, stage_id == num_stages - 1
        model.flatten()
        self.profiling = False
        self.fwd_ns: List[int] = []
        self.bwd_ns: List[int] = []
        self._saved = {}
        self._inflight = []
        self.loss_sum = None

    # ---- configuration
    def set_num_microbatches(self, m):
        self.num_microbatches = max(1, int(m))

    def set_balance_weights(self, w):
        self.balance = list(w)
        self.lo, self.hi = split_model(self.model.cfg.num_layers, self.S, self.balance)[self.sid]

    def set_profiling(self, on: bool):
        self.profiling = on

    def print_profile(self):
        f = sum(self.fwd_ns) / max(1, len(self.fwd_ns)) / 1e6
        b = sum(self.bwd_ns) / max(1, len(self.bwd_ns)) / 1e6
        print(f"stage {self.sid}: layers [{self.lo}, {self.hi}) forward {f:.3f} ms backward {b:.3f} ms per micro-batch")

    def owned_layers(self):
        return list(range(self.lo, self.hi))

    # ---- transport
    def _send(self, t, dst):
        # non-blocking: in 1F1B neighbouring stages send to each other at the same time, and a blocking send on both
        # sides would wait for a receive that is never posted
        t = t.contiguous()
        self._inflight.append((dist.isend(t, self.stage_ranks[dst], group=self.ctx.group), t))

    def _drain(self):
        for h, _ in self._inflight:
            h.wait()
        self._inflight = []

    def _recv(self, shape, dtype, src, device):
        t = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(t, self.stage_ranks[src], group=self.ctx.group)
        return t

    # ---- one micro-batch
    @torch.no_grad()
    def forward_microbatch(self, mb: int, ids: torch.Tensor, labels: Optional[torch.Tensor] = None):
        """Runs this stage's layers on micro-batch ``mb``; keeps what backward needs."""
        t0 = time.perf_counter_ns()
        m, cfg = self.model, self.model.cfg
        B, S = ids.shape
        dev, dt = m.tok_embeddings.device, m.tok_embeddings.dtype
        h = m.embed(ids) if self.first else self._recv((B * S, cfg.hidden_size), dt, self.sid - 1, dev)
        rope = m.rope(dev)
        ctxs = []
        for i in range(self.lo, self.hi):
            h, c = block_forward(cfg, m.layers[i], h, B, S, rope, save=True)
            ctxs.append(c)
        self._saved[mb] = (ctxs, ids, labels, h if self.last else None)
        if not self.last:
            self._send(h, self.sid + 1)
        if self.profiling:
            self.fwd_ns.append(time.perf_counter_ns() - t0)
        return h

    @torch.no_grad()
    def backward_microbatch(self, mb: int, n_valid_total=None):
        t0 = time.perf_counter_ns()
        m, cfg = self.model, self.model.cfg
        ctxs, ids, labels, h_last = self._saved.pop(mb)
        dev, dt = m.tok_embeddings.device, m.tok_embeddings.dtype
        B, S = ids.shape
        rope = m.rope(dev)
        if self.last:
            loss, dh = m.head_loss_backward(h_last, labels.reshape(-1), n_valid=n_valid_total)
            self.loss_sum = loss if self.loss_sum is None else self.loss_sum + loss
        else:
            dh = self._recv((B * S, cfg.hidden_size), dt, self.sid + 1, dev)
        for i in range(self.hi - 1, self.lo - 1, -1):
            dh = block_backward(cfg, m.layers[i], ctxs[i - self.lo], dh, rope)
        if self.first:
            F.embedding_bwd(ids.reshape(-1), dh, m.tok_embeddings.main_grad,
                            m.pos_embeddings.main_grad if m.pos_embeddings is not None else None, S)
        else:
            self._send(dh, self.sid - 1)
        if self.profiling:
            self.bwd_ns.append(time.perf_counter_ns() - t0)

    # ---- schedules
    def _split(self, ids, labels):
        M = self.num_microbatches
        assert ids.shape[0] % M == 0, "batch must divide into the micro-batches"
        n_valid = (labels != -100).sum().clamp(min=1).float() if labels is not None else None
        return list(zip(ids.chunk(M), labels.chunk(M))), n_valid

    def run_gpipe(self, ids, labels):
        """All forwards, then all backwards.  Returns the mean loss on the last stage (None elsewhere)."""
        mbs, n_valid = self._split(ids, labels)
        self.loss_sum = None
        for k, (i, l) in enumerate(mbs):
            self.forward_microbatch(k, i, l)
        for k in reversed(range(len(mbs))):
            self.backward_microbatch(k, n_valid)
        self._drain()
        return self.loss_sum

    def run_1f1b(self, ids, labels):
        mbs, n_valid = self._split(ids, labels)
        M = len(mbs)
        self.loss_sum = None
        warm = min(M, self.S - 1 - self.sid)
        f = b = 0
        for _ in range(warm):
            self.forward_microbatch(f, *mbs[f])
            f += 1
        while f < M:                        # steady state
            self.forward_microbatch(f, *mbs[f])
            f += 1
            self.backward_microbatch(b, n_valid)
            b += 1
        while b < M:                        # cool-down
            self.backward_microbatch(b, n_valid)
            b += 1
        self._drain()
        return self.loss_sum

    forward_1f1b = run_1f1b

    def max_live_microbatches(self, schedule="1f1b"):
        """Activations a stage holds at once: GPipe M, 1F1B min(M, stages - stage_id)."""
        return self.num_microbatches if schedule == "gpipe" else min(self.num_microbatches, self.S - self.sid)

    def bubble_fraction(self):
        return (self.S - 1) / (self.num_microbatches + self.S - 1)

    def accumulated_gradient(self):
        return self.model.flat.grads

    def clear_accumulated_gradients(self):
        self.model.flat.zero_grad()

    def owned_parameters(self):
        """Parameters this stage updates (its layers, plus embedding / head on the end stages; a tied embedding is
        updated by both end stages, whose gradients must then be summed by the caller)."""
        ps = [p for i in range(self.lo, self.hi) for p in self.model.layers[i].parameters()]
        if self.first:
            ps.append(self.model.tok_embeddings)
        if self.last:
            ps += [self.model.norm] + ([] if self.model.cfg.tie_embeddings and self.first else [self.model.lm_head])
        return ps


class DualPipe:
    """Bidirectional pipeline slot table (bookkeeping only, like the reference skeleton): micro-batches enter from both
    ends; ``schedule()`` lists, per time step, which (direction, micro-batch, phase) each stage would run."""

    def __init__(self, num_stages: int, num_microbatches: int):
        self.S, self.M = num_stages, num_microbatches

    def schedule(self):
        steps = []
        half = (self.M + 1) // 2
        for t in range(half + self.S - 1):
            row = []
            for s in range(self.S):
                a, b = t - s, t - (self.S - 1 - s)
                slot = []
                if 0 <= a < half:
                    slot.append(("down", a, "F"))
                if 0 <= b < self.M - half:
                    slot.append(("up", half + b, "F"))
                row.append(slot)
            steps.append(row)
        return steps
