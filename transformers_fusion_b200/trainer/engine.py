"""Training step engine: the object the trainers and the benchmark drive.

One engine owns a model with flat parameter / gradient buffers, the sharded fused optimizer and the
data-parallel gradient path.  ``step(ids, labels)`` runs on device-resident batches and returns the
loss as a device scalar; ``train_step(ids_cpu, labels_cpu)`` is the end-to-end form (pinned host
batch -> device, step, loss back to the host).

Data-parallel modes (``zero_stage``):
  0  plain DDP semantics: gradients all-reduced, every rank updates everything
  1/2 ZeRO: gradients reduce-scattered, each rank updates its contiguous shard of the flat buffer,
     updated bf16 parameters all-gathered.  ``comm="fused"`` uses the peer-memory kernels
     (reduce-scatter fused with the 1/W scale and squared-norm partials; AdamW fused with the
     all-gather of the refreshed bf16 parameters); ``comm="nccl"`` is the library baseline.
With a static batch shape the whole step can be captured into one CUDA graph (``cuda_graph=True``).

Reference counterparts: DistributedDataParallel::sync_gradients / allreduce_bucket
(src/trainer/ddp.cpp:113-173), ZeroOptimizer::reduce_scatter_grads / all_gather_params
(src/trainer/zero_optimizer_core.cpp:173-298), Trainer::micro_step (src/trainer/trainer_core.cpp:533-814).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .fused_optim import FlatAdamW


class PendingLoss:
    """Loss of an enqueued step: a pinned host slot plus the event recorded after its device-to-host copy.  The slot is
    reused four steps later, so read the value before enqueuing the fourth step after this one."""

    def __init__(self, slot, event, value):
        self._slot, self._event, self._value = slot, event, value

    def ready(self) -> bool:
        return self._event is None or self._event.query()

    def value(self) -> float:
        if self._value is None:
            self._event.synchronize()
            self._value = float(self._slot[0])
        return self._value


class TrainEngine:
    def __init__(self, model, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0,
                 zero_stage=2, comm="fused", group=None, cuda_graph=False, grad_accum_steps=1, symm=None):
        self.model = model
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.zero_stage = zero_stage if self.world > 1 else 0
        self.comm = comm if self.world > 1 else "none"
        self.grad_accum_steps = max(1, int(grad_accum_steps))
        self.cuda_graph = cuda_graph
        self.symm = symm
        pad = self.world * 1024
        if symm is not None and model.flat is None:
            from ..models.dense import FlatBuffers
            model.flat = FlatBuffers(model, dtype=model.tok_embeddings.dtype, pad_to=pad, allocator=symm.alloc)
        self.flat = model.flatten(pad_to=pad)
        n = self.flat.numel
        if self.zero_stage >= 1:
            per = n // self.world
            self.shard = (self.rank * per, (self.rank + 1) * per)
        else:
            self.shard = (0, n)
        self.opt = FlatAdamW(self.flat, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                             max_grad_norm=max_grad_norm, shard=self.shard,
                             norm_reduce=self._norm_reduce if self.zero_stage >= 1 else None)
        self._graphs = {}            # {closes the accumulation window?: (graph, static inputs, static loss)}
        self._micro = 0
        self.launches_per_step = 0   # kernels inside the captured graph (0 while running eagerly)
        self.fused = None
        if self.comm == "fused":
            from ..parallel.zero_fused import FusedZero
            self.fused = FusedZero(self.flat, self.opt, symm, self.rank, self.world)

    # ------------------------------------------------------------------ gradient path
    def _norm_reduce(self, t):
        dist.all_reduce(t, group=self.group)

    def _sync_and_update(self):
        """Gradient reduction + optimizer update (hyper-parameters of this step are already staged)."""
        flat, opt = self.flat, self.opt
        if self.world == 1:
            opt.step(staged=True)
            return
        if self.comm == "fused":
            self.fused.step()
            return
        W = self.world
        if self.zero_stage == 0:
            flat.grads.div_(W)
            dist.all_reduce(flat.grads, group=self.group)
            opt.step(staged=True)
            return
        lo, hi = self.shard
        flat.grads.div_(W)
        shard = flat.grads[lo:hi]
        dist.reduce_scatter_tensor(shard, flat.grads, group=self.group)
        opt.step(staged=True)
        # the optimizer zeroes only its shard; the rest of the buffer must start the next step at zero too
        if lo > 0:
            flat.grads[:lo].zero_()
        if hi < flat.numel:
            flat.grads[hi:].zero_()
        dist.all_gather_into_tensor(flat.params, flat.params[lo:hi].clone(), group=self.group)

    # ------------------------------------------------------------------ steps
    def _step_impl(self, ids, labels, final=True):
        """Forward + backward of one micro-batch (gradients scaled by 1 / grad_accum_steps and added to the flat buffer);
        the reduction and the optimizer update follow only on the micro-batch that closes the accumulation window."""
        loss = self.model.forward_backward(ids, labels, loss_scale=1.0 / self.grad_accum_steps)
        if final:
            self._sync_and_update()
        return loss

    def _capture(self, final, ids, labels):
        """Warm-up on a side stream (allocator pools, lazy kernel attribute calls), then capture.  The warm-up is a real
        step, so the training state is put back afterwards."""
        opt = self.opt
        static = (ids.clone(), labels.clone())
        state = (self.flat.params, opt.master, opt.m, opt.v, self.flat.grads)
        snap = [t.clone() for t in state]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._step_impl(*static, final=final)
        torch.cuda.current_stream().wait_stream(s)
        for dst, src in zip(state, snap):
            dst.copy_(src)
        del snap
        from ..ops import _lib
        graph = torch.cuda.CUDAGraph()
        n0 = _lib.LAUNCHES[0]
        with torch.cuda.graph(graph):
            loss = self._step_impl(*static, final=final)
        if final:
            self.launches_per_step = _lib.LAUNCHES[0] - n0
        return graph, static, loss

    def step(self, ids, labels, lr=None):
        """One micro-batch on a device-resident batch; every ``grad_accum_steps``-th call reduces the accumulated
        gradients and applies the optimizer update.  Returns the local mean loss of the micro-batch (device scalar)."""
        self._micro += 1
        final = self._micro % self.grad_accum_steps == 0
        if not self.cuda_graph or not ids.is_cuda:
            if final:
                self.opt.stage_hyper(lr)
            return self._step_impl(ids, labels, final)
        if self._graphs.get(final) is None:
            if final:
                self.opt.stage_hyper(lr)       # the warm-up step reads staged values; it does not count as a step
                self.opt.step_count -= 1
            self._graphs[final] = self._capture(final, ids, labels)
        graph, static, loss = self._graphs[final]
        if final:
            self.opt.stage_hyper(lr)
        static[0].copy_(ids, non_blocking=True)
        static[1].copy_(labels, non_blocking=True)
        graph.replay()
        return loss

    def train_step(self, ids_cpu, labels_cpu, lr=None) -> float:
        """End-to-end step: pinned host batch -> device -> step -> loss on the host (waits for the step)."""
        return self.train_step_async(ids_cpu, labels_cpu, lr).value()

    def train_step_async(self, ids_cpu, labels_cpu, lr=None) -> "PendingLoss":
        """End-to-end step without stalling the host: the batch is copied from (pinned) host memory, the step is enqueued
        and the loss is copied back into a pinned slot behind an event.  ``value()`` on the returned handle waits for that
        event only, so a loop that reads the loss of step i after enqueuing step i + 1 keeps the device busy while still
        reading every step's loss."""
        dev = self.flat.params.device
        ids = ids_cpu.to(dev, non_blocking=True)
        labels = labels_cpu.to(dev, non_blocking=True)
        loss = self.step(ids, labels, lr)
        if not loss.is_cuda:
            return PendingLoss(None, None, float(loss))
        if getattr(self, "_loss_ring", None) is None:
            self._loss_ring = [(torch.empty(1, dtype=torch.float32).pin_memory(), torch.cuda.Event()) for _ in range(4)]
            self._loss_slot = 0
        slot, ev = self._loss_ring[self._loss_slot]
        self._loss_slot = (self._loss_slot + 1) % len(self._loss_ring)
        slot.copy_(loss.detach().reshape(1).float(), non_blocking=True)
        ev.record()
        return PendingLoss(slot, ev, None)
