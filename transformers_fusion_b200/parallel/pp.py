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
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..models.dense import _norm_fwd, block_backward, block_forward
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


@dataclass
class PipelineStage:
    device_id: int
    layer_start: int
    layer_end: int
    model_segment: object


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
        self.loss_sum = None

    # ---- configuration
    def context(self) -> DistributedContext:
        return self.ctx

    def stage(self) -> "PipelineStage":
        """What this rank owns: its device, the half-open layer range and the model (whose other layers are never run)."""
        dev = self.model.tok_embeddings.device
        return PipelineStage(dev.index if dev.type == "cuda" and dev.index is not None else 0, self.lo, self.hi, self.model)

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
    def _exchange(self, send_next=None, send_prev=None, recv_next=None, recv_prev=None):
        """Point-to-point traffic of one schedule slot, posted as ONE batch (``dist.batch_isend_irecv``) and waited for.

        Pairing a slot's send with its receive matters on NCCL: neighbouring stages share one communicator, so a send
        and a receive enqueued as separate calls run in program order, and in the steady state of 1F1B stage s wants to
        send activations while stage s + 1 wants to send gradients; each would wait for a receive that the other has
        queued behind its own send.  Inside one batch NCCL progresses all of the operations together.
        ``recv_next`` / ``recv_prev`` are (shape, dtype, device) of the tensor expected from that neighbour."""
        ops, got_next, got_prev, keep = [], None, None, []
        nxt = self.stage_ranks[self.sid + 1] if self.sid + 1 < self.S else None
        prv = self.stage_ranks[self.sid - 1] if self.sid > 0 else None
        if send_prev is not None:
            keep.append(send_prev.contiguous())
            ops.append(dist.P2POp(dist.isend, keep[-1], prv, group=self.ctx.group))
        if recv_prev is not None:
            got_prev = torch.empty(recv_prev[0], dtype=recv_prev[1], device=recv_prev[2])
            ops.append(dist.P2POp(dist.irecv, got_prev, prv, group=self.ctx.group))
        if send_next is not None:
            keep.append(send_next.contiguous())
            ops.append(dist.P2POp(dist.isend, keep[-1], nxt, group=self.ctx.group))
        if recv_next is not None:
            got_next = torch.empty(recv_next[0], dtype=recv_next[1], device=recv_next[2])
            ops.append(dist.P2POp(dist.irecv, got_next, nxt, group=self.ctx.group))
        if ops:
            for h in dist.batch_isend_irecv(ops):
                h.wait()
        return got_next, got_prev

    def _hidden_spec(self, ids):
        m = self.model
        return ((ids.shape[0] * ids.shape[1], m.cfg.hidden_size), m.tok_embeddings.dtype, m.tok_embeddings.device)

    # ---- one micro-batch (compute only; the schedules move the tensors)
    @torch.no_grad()
    def forward_microbatch(self, mb: int, ids: torch.Tensor, labels: Optional[torch.Tensor] = None, h_in=None):
        """Runs this stage's layers on micro-batch ``mb`` (``h_in`` = hidden state received from the previous stage;
        the first stage embeds ``ids``); keeps what backward needs and returns the stage's output."""
        t0 = time.perf_counter_ns()
        m, cfg = self.model, self.model.cfg
        B, S = ids.shape
        dev = m.tok_embeddings.device
        h = m.embed(ids) if self.first else h_in
        rope = m.rope(dev)
        ctxs = []
        for i in range(self.lo, self.hi):
            h, c = block_forward(cfg, m.layers[i], h, B, S, rope, save=True)
            ctxs.append(c)
        self._saved[mb] = (ctxs, ids, labels, h if self.last else None)
        if self.profiling:
            self.fwd_ns.append(time.perf_counter_ns() - t0)
        return h

    @torch.no_grad()
    def backward_microbatch(self, mb: int, n_valid_total=None, dh=None):
        """Backward of micro-batch ``mb`` (``dh`` = gradient received from the next stage; the last stage starts from
        the loss).  Returns the gradient for the previous stage (None on the first stage)."""
        t0 = time.perf_counter_ns()
        m, cfg = self.model, self.model.cfg
        ctxs, ids, labels, h_last = self._saved.pop(mb)
        dev = m.tok_embeddings.device
        B, S = ids.shape
        rope = m.rope(dev)
        if self.last:
            loss, dh = m.head_loss_backward(h_last, labels.reshape(-1), n_valid=n_valid_total)
            self.loss_sum = loss if self.loss_sum is None else self.loss_sum + loss
        for i in range(self.hi - 1, self.lo - 1, -1):
            dh = block_backward(cfg, m.layers[i], ctxs[i - self.lo], dh, rope)
        if self.first:
            F.embedding_bwd(ids.reshape(-1), dh, m.tok_embeddings.main_grad,
                            m.pos_embeddings.main_grad if m.pos_embeddings is not None else None, S)
            dh = None
        if self.profiling:
            self.bwd_ns.append(time.perf_counter_ns() - t0)
        return dh

    # ---- schedules
    def _split(self, ids, labels):
        M = self.num_microbatches
        assert ids.shape[0] % M == 0, "batch must divide into the micro-batches"
        n_valid = (labels != -100).sum().clamp(min=1).float() if labels is not None else None
        return list(zip(ids.chunk(M), labels.chunk(M))), n_valid

    def run_gpipe(self, ids, labels):
        """All forwards, then all backwards.  Returns the mean loss on the last stage (None elsewhere)."""
        mbs, n_valid = self._split(ids, labels)
        spec = self._hidden_spec(mbs[0][0])
        self.loss_sum = None
        for k, (i, l) in enumerate(mbs):
            h_in = None if self.first else self._exchange(recv_prev=spec)[1]
            h = self.forward_microbatch(k, i, l, h_in)
            if not self.last:
                self._exchange(send_next=h)
        for k in reversed(range(len(mbs))):
            dh = None if self.last else self._exchange(recv_next=spec)[0]
            d_in = self.backward_microbatch(k, n_valid, dh)
            if not self.first:
                self._exchange(send_prev=d_in)
        self._finish()
        return self.loss_sum

    def run_1f1b(self, ids, labels):
        """Warm-up forwards, steady one-forward-one-backward, cool-down backwards.  In the steady state the activation
        that goes to the next stage and the gradient that comes back from it travel in one batch, and so do the
        gradient for the previous stage and the next activation from it."""
        mbs, n_valid = self._split(ids, labels)
        M = len(mbs)
        spec = self._hidden_spec(mbs[0][0])
        self.loss_sum = None
        warm = min(M, self.S - 1 - self.sid)
        steady = M - warm
        for k in range(warm):
            h_in = None if self.first else self._exchange(recv_prev=spec)[1]
            h = self.forward_microbatch(k, *mbs[k], h_in)
            if not self.last:
                self._exchange(send_next=h)
        h_in = None
        if steady > 0 and not self.first:
            h_in = self._exchange(recv_prev=spec)[1]
        for k in range(steady):
            h = self.forward_microbatch(warm + k, *mbs[warm + k], h_in)
            dh = None
            if not self.last:
                dh = self._exchange(send_next=h, recv_next=spec)[0]
            d_in = self.backward_microbatch(k, n_valid, dh)
            if not self.first:
                more = k + 1 < steady
                h_in = self._exchange(send_prev=d_in, recv_prev=spec if more else None)[1]
        for k in range(steady, M):                          # cool-down
            dh = None if self.last else self._exchange(recv_next=spec)[0]
            d_in = self.backward_microbatch(k, n_valid, dh)
            if not self.first:
                self._exchange(send_prev=d_in)
        self._finish()
        return self.loss_sum

    def _finish(self):
        """End of a schedule: a tied embedding has one copy on the first stage (embedding gradient) and one on the last
        (LM-head gradient); both copies must see the sum, or they drift apart."""
        if self.model.cfg.tie_embeddings and self.S > 1 and (self.first or self.last):
            g = self.model.tok_embeddings.main_grad
            other = self.stage_ranks[-1] if self.first else self.stage_ranks[0]
            buf = torch.empty_like(g)
            ops = [dist.P2POp(dist.isend, g, other, group=self.ctx.group), dist.P2POp(dist.irecv, buf, other, group=self.ctx.group)]
            for h in dist.batch_isend_irecv(ops):
                h.wait()
            g.add_(buf)

    def grad_norm(self) -> float:
        """Global gradient norm over all stages (every stage returns the same value); a tied embedding counts once."""
        skip = self.model.tok_embeddings if (self.model.cfg.tie_embeddings and self.S > 1 and self.last) else None
        sq = torch.zeros(1, dtype=torch.float32, device=self.model.tok_embeddings.device)
        for p in self.owned_parameters():
            if p is not skip:
                sq += p.main_grad.float().pow(2).sum()
        if self.S > 1:
            dist.all_reduce(sq, group=self.ctx.group)
        return float(sq.sqrt())

    def clip_gradients(self, max_norm: float) -> float:
        """Scales this stage's gradients by the factor that brings the GLOBAL norm to ``max_norm``."""
        norm = self.grad_norm()
        if max_norm > 0 and norm > max_norm:
            seen = set()
            for p in self.owned_parameters():
                if id(p) not in seen:
                    seen.add(id(p))
                    p.main_grad.mul_(max_norm / (norm + 1e-6))
        return norm

    def forward_1f1b(self, ids, labels):
        """The reference splits 1F1B into a forward and a backward call (pipeline.h:42-45); here the schedule interleaves
        them, so this call runs all of it and ``backward_1f1b`` reports its result."""
        self._last_loss = self.run_1f1b(ids, labels)
        return self._last_loss

    def backward_1f1b(self):
        """Loss of the schedule run by ``forward_1f1b`` (last stage; None elsewhere).  The gradients are already
        accumulated in ``accumulated_gradient()``."""
        return getattr(self, "_last_loss", None)

    @torch.no_grad()
    def forward(self, ids):
        """Inference pass through the pipeline: every stage runs its layers on the whole batch and hands the hidden state
        to the next one; the last stage returns the logits [B, S, V] (the other stages return None)."""
        m, cfg = self.model, self.model.cfg
        B, S = ids.shape
        h = m.embed(ids) if self.first else self._exchange(recv_prev=self._hidden_spec(ids))[1]
        rope = m.rope(m.tok_embeddings.device)
        for i in range(self.lo, self.hi):
            h, _ = block_forward(cfg, m.layers[i], h, B, S, rope, save=False)
        if not self.last:
            self._exchange(send_next=h)
            return None
        f, _ = _norm_fwd(cfg, h, m.norm, m.norm_bias)
        return F.gemm(f, m.lm_head.data).view(B, S, -1)

    @staticmethod
    def compute_loss(logits, labels, ignore_index: int = -100):
        """Mean cross entropy of logits [B, S, V] (or [T, V]) against labels."""
        return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1),
                                                 ignore_index=ignore_index)

    def num_micro_batches(self) -> int: return self.num_microbatches
    def micro_batch_queue_size(self) -> int: return len(self._saved)
    def balance_weights(self): return list(self.balance) if self.balance else []

    def model_param_count(self) -> int:
        """Parameters this stage owns (a tied embedding is counted on both end stages, which both hold a copy)."""
        seen, n = set(), 0
        for p in self.owned_parameters():
            if id(p) not in seen:
                seen.add(id(p))
                n += p.numel()
        return n

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
        updated by both end stages from the summed gradient that the schedules leave on both of them)."""
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
