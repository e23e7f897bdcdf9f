"""Collective communication.

* ``DistributedContext`` - rank / world bookkeeping and all_reduce / broadcast / all_gather / barrier on tensors, over
  ``torch.distributed`` (NCCL on GPUs, gloo on CPU).  ``DistributedContext.init()`` reads the torchrun environment.
* ``SymmCollectives``    - the same collectives as single fused kernels over symmetric peer memory (one-shot and
  two-shot all-reduce, reduce-scatter, all-gather, broadcast; bf16 / fp32; sum / avg / max / min), for the
  latency-bound sizes of tensor-parallel decode.  Bounded waits; errors surface through the status word.
* ``RingAllReduce``      - the reference's API (allreduce with ops, chunked variant, reduce_scatter, allgather, scatter,
  gather, hierarchical_allreduce).  There is no ring on NVSwitch: calls map onto SymmCollectives when a symmetric heap
  is attached and onto torch.distributed otherwise.
* ``ParameterServer``    - sharded key/value store of tensors with versioning and stale-gradient damping.

Reference counterparts: src/trainer/distributed.cpp (DistributedContext :21-123, RingAllReduce :288-591,
ParameterServer :597-885)."""
from __future__ import annotations

import os
import threading
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

OPS = {"sum": 0, "avg": 1, "max": 2, "min": 3}
_TORCH_OPS = {"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}


class DistributedContext:
    def __init__(self, rank: int = 0, world_size: int = 1, group=None):
        self.rank, self.world_size, self.group = rank, world_size, group

    @classmethod
    def init(cls, backend: Optional[str] = None, timeout_s: float = 600.0) -> "DistributedContext":
        """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (single process when unset)."""
        import datetime
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        if world > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29500")
            if backend is None:
                backend = "nccl" if torch.cuda.is_available() else "gloo"
            if backend == "nccl":
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
            dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
        return cls(rank, world)

    @property
    def is_distributed(self):
        return self.world_size > 1 and dist.is_initialized()

    @property
    def world_rank(self) -> int:
        return self.rank

    #: how the ranks of this context cooperate ("DDP", "TENSOR_PARALLEL", "PIPELINE_PARALLEL"); informational
    mode: str = "DDP"

    def is_main(self) -> bool:
        return self.rank == 0

    def all_reduce(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if self.is_distributed:
            dist.all_reduce(t, op=_TORCH_OPS[op], group=self.group)
            if op == "avg":
                t.div_(self.world_size)
        return t

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        if self.is_distributed:
            dist.broadcast(t, src=root, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenation of every rank's ``t`` along dim 0."""
        if not self.is_distributed:
            return t.clone()
        out = torch.empty((self.world_size * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def reduce_scatter(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """This rank's 1/W slice (dim 0) of the reduction of ``t`` over ranks."""
        if not self.is_distributed:
            return t.clone()
        n = t.shape[0] // self.world_size
        out = torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        if dist.get_backend(self.group) == "gloo":      # gloo has no reduce_scatter: reduce, then slice
            full = t.clone()
            dist.all_reduce(full, op=_TORCH_OPS[op], group=self.group)
            out.copy_(full[self.rank * n:(self.rank + 1) * n])
        else:
            dist.reduce_scatter_tensor(out, t.contiguous(), op=_TORCH_OPS[op], group=self.group)
        if op == "avg":
            out.div_(self.world_size)
        return out

    def barrier(self):
        if self.is_distributed:
            dist.barrier(group=self.group)

    def send(self, t, dst, tag=0):
        dist.send(t.contiguous(), dst, group=self.group, tag=tag)

    def recv(self, t, src, tag=0):
        dist.recv(t, src, group=self.group, tag=tag)
        return t


class SymmCollectives:
    """Fused collectives on staging buffers in symmetric memory (``capacity`` bytes per rank each).

    There are two staging buffers and consecutive collectives alternate between them.  That lets the one-shot all-reduce
    run without its closing barrier: a rank leaves the opening barrier of collective n+1 only after every peer has
    finished collective n, so by the time a buffer is refilled (collective n+2) nobody reads it.  The alternation is
    host-side state, so a sequence that is replayed (a CUDA graph) must hold an even number of collectives and start on
    the buffer it was captured on: capture_begin / capture_end / before_replay take care of both."""

    def __init__(self, symm, capacity_bytes: int = 8 << 20):
        from ..ops import _lib
        self._lib = _lib
        _lib.register("tfb_collective", [_lib.c_p, _lib.c_p, _lib.c_ll, _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_i, _lib.c_p, _lib.c_p,
                                         _lib.c_i, _lib.c_i, _lib.c_p, _lib.c_p, _lib.c_i, _lib.c_p, _lib.c_i, _lib.c_p])
        self.symm, self.rank, self.world = symm, symm.rank, symm.world
        gran = 16 * self.world
        self.capacity = (capacity_bytes + gran - 1) // gran * gran
        self._stages = [symm.alloc_bytes(self.capacity), symm.alloc_bytes(self.capacity)]
        self._half = 0
        self.count = 0                  # collectives launched (or captured) so far
        self.ticket = torch.zeros(1, dtype=torch.int32, device=symm.device)
        symm.on_reset(self.ticket.zero_)
        self.one_shot_max_bytes = 256 << 10
        # flag-in-data all-reduce: receive area [2 parities][world senders][one_shot_max_bytes of data as 8-byte pairs]
        _lib.register("tfb_allreduce_ll", [_lib.c_p, _lib.c_p, _lib.c_p, _lib.c_p, _lib.c_ll, _lib.c_ll, _lib.c_i, _lib.c_i, _lib.c_i,
                                           _lib.c_i, _lib.c_p, _lib.c_p, _lib.c_p, _lib.c_i, _lib.c_p])
        self._ll_recv = symm.alloc_bytes(2 * self.world * self.one_shot_max_bytes * 2)
        self._ll_state = torch.zeros(2, dtype=torch.int32, device=symm.device)      # sequence number, ticket

        def _ll_clear():
            self._ll_recv.view(torch.int32, self._ll_recv.nbytes // 4).zero_()
            self._ll_state.zero_()
        _ll_clear()
        symm.on_reset(_ll_clear)
        symm.barrier()                  # nobody pushes into an area that its owner has not cleared yet

    @property
    def stage(self):
        """The staging buffer the next collective works on."""
        return self._stages[self._half]

    def _run(self, local, n, dtype, op, mode, root=0, max_ctas=0, extra=None, open_ended=False):
        lib, s = self._lib, self.symm
        lib.check(lib.lib().tfb_collective(self.stage.ptrs.data_ptr(), lib.ptr(local), n, 0 if dtype == torch.bfloat16 else 1, OPS[op],
                                           mode, root, s.flags.ptrs.data_ptr(), s.epoch.data_ptr(), self.rank, self.world,
                                           lib.status_word(s.device).data_ptr(), self.ticket.data_ptr(), max_ctas,
                                           lib.ptr(extra), 1 if open_ended else 0, lib.stream()),
                  "collective")
        self._half ^= 1
        self.count += 1

    def _pad(self):
        """One smallest collective (with its closing barrier): moves the alternation on by one."""
        n = 16 * self.world // 4
        self._run(torch.empty(n, dtype=torch.float32, device=self.symm.device), n, torch.float32, "sum", 0, max_ctas=1)

    # A captured sequence has its staging buffers baked in.  capture_begin() notes which buffer it starts on,
    # capture_end() (still inside the capture) makes the number of captured collectives even, so that the sequence ends
    # on the other buffer, and before_replay() brings the host-side alternation to the captured starting point (with one
    # small eager collective when the eager work in between left it on the other buffer).
    def capture_begin(self):
        return (self._half, self.count)

    def capture_end(self, token):
        if (self.count - token[1]) & 1:
            self._pad()

    def before_replay(self, token):
        if self._half != token[0]:
            self._pad()

    def _padded(self, t):
        assert t.dtype in (torch.bfloat16, torch.float32) and t.is_contiguous()
        esz = t.element_size()
        gran = 16 * self.world // esz
        n = (t.numel() + gran - 1) // gran * gran
        assert n * esz <= self.capacity, "message exceeds the staging buffer"
        return n

    def all_reduce(self, t: torch.Tensor, op="sum", algo="auto") -> torch.Tensor:
        """In place on ``t``.  ``algo``: one_shot | two_shot | auto (by size)."""
        nb = t.numel() * t.element_size()
        if algo == "auto" and nb <= self.one_shot_max_bytes and nb % 16 == 0 and t.data_ptr() % 16 == 0:
            return self.all_reduce_ll(t, op, out=t)       # no staging copy, no barrier
        n = self._padded(t)
        st = self.stage.view(t.dtype, n)
        st[: t.numel()].copy_(t.reshape(-1))
        if n > t.numel():
            st[t.numel():].zero_()
        one = algo == "one_shot" or (algo == "auto" and n * t.element_size() <= self.one_shot_max_bytes)
        if one:
            if n == t.numel():
                self._run(t, n, t.dtype, op, 0, max_ctas=self._one_shot_ctas(n * t.element_size()), open_ended=True)
            else:
                out = torch.empty(n, dtype=t.dtype, device=t.device)
                self._run(out, n, t.dtype, op, 0, max_ctas=self._one_shot_ctas(n * t.element_size()), open_ended=True)
                t.copy_(out[: t.numel()].view(t.shape))
        else:
            self._run(None, n, t.dtype, op, 1)
            t.copy_(st[: t.numel()].view(t.shape))
        return t

    @staticmethod
    def _one_shot_ctas(nbytes: int) -> int:
        """One CTA up to 8 KiB (the barrier is paid once), then one per 16 KiB up to 32."""
        return max(1, min(32, nbytes // (16 << 10)))

    def all_reduce_ll(self, x: torch.Tensor, op="sum", residual: Optional[torch.Tensor] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Latency-bound all-reduce of a local tensor (any local memory; at most ``one_shot_max_bytes``, a multiple of 16
        bytes): every rank pushes its data, tagged with a sequence number, into the peers' receive areas and reduces what
        arrives in its own - no barrier, nothing host-side to keep in step (safe in captured graphs).  ``residual``: local
        addend (op sum).  Result in ``out`` (default: a new tensor; may be ``x`` itself)."""
        assert x.is_contiguous() and x.dtype in (torch.bfloat16, torch.float32)
        nbytes = x.numel() * x.element_size()
        assert nbytes % 16 == 0 and nbytes <= self.one_shot_max_bytes, "message not a multiple of 16 bytes or too large"
        if out is None:
            out = torch.empty_like(x)
        if residual is not None:
            assert op == "sum" and residual.dtype == x.dtype and residual.numel() == x.numel() and residual.is_contiguous()
        lib = self._lib
        lib.check(lib.lib().tfb_allreduce_ll(self._ll_recv.ptrs.data_ptr(), x.data_ptr(), lib.ptr(residual), out.data_ptr(), x.numel(),
                                             self.one_shot_max_bytes, 0 if x.dtype == torch.bfloat16 else 1, OPS[op], self.rank,
                                             self.world, self._ll_state.data_ptr(), self._ll_state[1:].data_ptr(),
                                             lib.status_word(self.symm.device).data_ptr(), 0, lib.stream()), "allreduce_ll")
        return out

    def stage_view(self, dtype, numel: int):
        """View of this rank's staging buffer for producers that write their result there directly (saves the copy-in of
        all_reduce); None when ``numel`` does not fit or is not a whole number of 16-byte x world granules."""
        esz = torch.empty(0, dtype=dtype).element_size()
        if numel * esz > self.capacity or (numel * esz) % (16 * self.world):
            return None
        return self.stage.view(dtype, numel)

    def all_reduce_staged(self, numel: int, dtype, op="sum", residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """All-reduce of data already in the staging buffer (see stage_view).  Returns a flat tensor holding the result:
        a fresh buffer for the one-shot form, the staging buffer itself for the two-shot form (consume it before the
        collective after the next one).  ``residual`` (same dtype, ``numel`` elements, op sum): added to the result -
        inside the kernel, before the one rounding, for the one-shot form."""
        esz = torch.empty(0, dtype=dtype).element_size()
        if residual is not None:
            assert op == "sum" and residual.dtype == dtype and residual.numel() == numel
            residual = residual.contiguous()
        if numel * esz <= self.one_shot_max_bytes:
            out = torch.empty(numel, dtype=dtype, device=self.symm.device)
            fuse = residual is not None and residual.data_ptr() % 16 == 0
            self._run(out, numel, dtype, op, 0, max_ctas=self._one_shot_ctas(numel * esz), extra=residual if fuse else None,
                      open_ended=True)
            if residual is not None and not fuse:
                out += residual.view(-1)
            return out
        st = self.stage.view(dtype, numel)
        self._run(None, numel, dtype, op, 1)
        return st if residual is None else st + residual.view(-1)

    def reduce_scatter(self, t: torch.Tensor, op="sum") -> torch.Tensor:
        n = self._padded(t)
        assert n == t.numel(), "reduce_scatter needs numel * elem_size to be a multiple of 16 * world"
        self.stage.view(t.dtype, n).copy_(t.reshape(-1))
        out = torch.empty(n // self.world, dtype=t.dtype, device=t.device)
        self._run(out, n, t.dtype, op, 2)
        return out

    def all_gather(self, shard: torch.Tensor) -> torch.Tensor:
        n = shard.numel() * self.world
        assert n * shard.element_size() % (16 * self.world) == 0 and n * shard.element_size() <= self.capacity
        st = self.stage.view(shard.dtype, n)
        self._run(shard.contiguous(), n, shard.dtype, "sum", 3)
        return st.clone()

    def broadcast(self, t: torch.Tensor, root=0) -> torch.Tensor:
        n = self._padded(t)
        st = self.stage.view(t.dtype, n)
        if self.rank == root:
            st[: t.numel()].copy_(t.reshape(-1))
        self._run(None, n, t.dtype, "sum", 4, root)
        t.copy_(st[: t.numel()].view(t.shape))
        return t


class RingAllReduce:
    """Reference-shaped facade (ops SUM / AVG / MAX / MIN; chunked and hierarchical variants keep their names)."""

    def __init__(self, ctx: DistributedContext, symm_collectives: Optional[SymmCollectives] = None):
        self.ctx, self.sc = ctx, symm_collectives

    def _dev(self, t):
        return self.sc is not None and t.is_cuda and t.dtype in (torch.bfloat16, torch.float32) and \
            t.numel() * t.element_size() <= self.sc.capacity - 16 * self.sc.world

    def world_size(self) -> int: return self.ctx.world_size
    def rank(self) -> int: return self.ctx.rank
    def barrier(self): self.ctx.barrier()

    def allreduce(self, t, op="sum"):
        return self.sc.all_reduce(t.contiguous(), op) if self._dev(t) else self.ctx.all_reduce(t, op)

    def allreduce_chunked(self, t, op="sum", chunk_elems=1 << 20):
        flat = t.reshape(-1)
        for o in range(0, flat.numel(), chunk_elems):
            seg = flat[o:o + chunk_elems]
            seg.copy_(self.allreduce(seg.clone(), op))
        return t

    allreduce_double_buffer = allreduce_chunked

    def reduce_scatter(self, t, op="sum"):
        return self.ctx.reduce_scatter(t, op)

    def allgather(self, t):
        return self.ctx.all_gather(t)

    def scatter(self, t, root=0):
        """Rank r receives slice r (dim 0) of the root's tensor."""
        full = self.ctx.broadcast(t.clone(), root)
        n = full.shape[0] // self.ctx.world_size
        return full[self.ctx.rank * n:(self.ctx.rank + 1) * n].clone()

    def gather(self, t, root=0):
        full = self.ctx.all_gather(t)
        return full if self.ctx.rank == root else None

    def hierarchical_allreduce(self, t, op="sum", inter_node_fn=None):
        """Intra-node reduction, then ``inter_node_fn(tensor)`` (e.g. an NCCL all-reduce over the node leaders' group).
        One NVSwitch domain is flat, so without an inter-node callback this is a plain all-reduce."""
        t = self.allreduce(t, op)
        if inter_node_fn is not None:
            t = inter_node_fn(t)
        return t


class ParameterServer:
    """Sharded tensor store (shard = hash(key) % num_shards) with versions.  ``update_gradient`` applies
    p -= lr * g; a gradient computed against an older version is damped (x0.5 when <= 5 versions stale, dropped
    beyond ``max_staleness``); pending updates are queued (bounded) and applied by a worker thread in async mode."""

    def __init__(self, num_shards=4, lr=0.01, max_queue=64, max_staleness=5, async_mode=False):
        self.num_shards, self.lr, self.max_queue, self.max_staleness = num_shards, lr, max_queue, max_staleness
        self.shards: List[Dict[str, torch.Tensor]] = [dict() for _ in range(num_shards)]
        self.versions: Dict[str, int] = {}
        self.lock = threading.Lock()
        self.queue: List = []
        self.dropped = 0
        self.async_mode = async_mode
        self._stop = False
        self._worker = None
        if async_mode:
            self._cv = threading.Condition(self.lock)
            self._worker = threading.Thread(target=self._loop, daemon=True)
            self._worker.start()

    def _shard(self, key):
        import zlib
        return self.shards[zlib.crc32(key.encode()) % self.num_shards]

    def push(self, key, t):
        with self.lock:
            self._shard(key)[key] = t.detach().clone()
            self.versions[key] = self.versions.get(key, 0) + 1

    def pull(self, key):
        with self.lock:
            return self._shard(key)[key].clone(), self.versions[key]

    def _apply(self, key, grad, version):
        stale = self.versions[key] - version
        if stale > self.max_staleness:
            self.dropped += 1
            return False
        scale = 0.5 if stale > 0 else 1.0
        self._shard(key)[key].add_(grad, alpha=-self.lr * scale)
        self.versions[key] += 1
        return True

    def update_gradient(self, key, grad, version):
        with self.lock:
            if not self.async_mode:
                return self._apply(key, grad, version)
            if len(self.queue) >= self.max_queue:
                self.dropped += 1
                return False
            self.queue.append((key, grad.detach().clone(), version))
            self._cv.notify()
            return True

    def _loop(self):
        while True:
            with self._cv:
                while not self.queue and not self._stop:
                    self._cv.wait(0.05)
                if self._stop and not self.queue:
                    return
                self._apply(*self.queue.pop(0))

    def flush(self):
        while True:
            with self.lock:
                if not self.queue:
                    return

    # ---- the reference's surface (include/quant/distributed.h: ParameterServer) ----------------------------------
    def configure_world(self, world_size: int, world_rank: int, num_ps_nodes: Optional[int] = None):
        """Describe the job this store is part of: the first ``num_ps_nodes`` ranks hold the shards."""
        self._world = (int(world_size), int(world_rank), int(num_ps_nodes or self.num_shards))
        return self

    def world_size(self) -> int: return getattr(self, "_world", (1, 0, self.num_shards))[0]
    def world_rank(self) -> int: return getattr(self, "_world", (1, 0, self.num_shards))[1]
    def num_ps_nodes(self) -> int: return getattr(self, "_world", (1, 0, self.num_shards))[2]
    def ps_node_id(self) -> int: return self.world_rank() if self.is_ps_node() else -1
    def is_ps_node(self) -> bool: return self.world_rank() < self.num_ps_nodes()

    @staticmethod
    def shard_for(name: str, num_ps_nodes: int) -> int:
        import zlib
        return zlib.crc32(name.encode()) % max(1, num_ps_nodes)

    def owns_param(self, name: str) -> bool:
        return name in self._shard(name)

    def get_param(self, name: str):
        with self.lock:
            t = self._shard(name).get(name)
            return None if t is None else t.clone()

    def list_params(self) -> List[str]:
        with self.lock:
            return sorted(k for sh in self.shards for k in sh)

    def remove_param(self, name: str):
        with self.lock:
            self._shard(name).pop(name, None)
            self.versions.pop(name, None)

    def clear_params(self):
        with self.lock:
            for sh in self.shards:
                sh.clear()
            self.versions.clear()

    def get_version(self, name: str) -> int:
        return self.versions.get(name, -1)

    def set_max_stale_gradients(self, n: int):
        self.max_staleness = int(n)

    def apply_weight_decay(self, decay_rate: float):
        with self.lock:
            for sh in self.shards:
                for t in sh.values():
                    t.mul_(1.0 - decay_rate)

    def average_parameters(self, weight: float = 1.0, ctx: Optional["DistributedContext"] = None):
        """Blend every stored tensor towards its mean over the ranks of ``ctx``: p <- (1 - weight) p + weight mean(p)."""
        if ctx is None or not ctx.is_distributed:
            return
        with self.lock:
            for sh in self.shards:
                for t in sh.values():
                    mean = ctx.all_reduce(t.clone(), "avg")
                    t.mul_(1.0 - weight).add_(mean, alpha=weight)

    def apply_momentum(self, momentum: float, lr: float):
        """One heavy-ball step from the gradients accumulated by ``accumulate_gradient``: v <- momentum v + g; p -= lr v."""
        with self.lock:
            vel = self.__dict__.setdefault("_velocity", {})
            for name, g in self.__dict__.setdefault("_grad_acc", {}).items():
                p = self._shard(name).get(name)
                if p is None:
                    continue
                v = vel.setdefault(name, torch.zeros_like(p))
                v.mul_(momentum).add_(g)
                p.add_(v, alpha=-lr)
                self.versions[name] += 1
            self._grad_acc = {}

    def accumulate_gradient(self, name: str, grad: torch.Tensor):
        with self.lock:
            acc = self.__dict__.setdefault("_grad_acc", {})
            acc[name] = acc[name] + grad if name in acc else grad.detach().clone()

    def push_async(self, key, t):
        """Queue a ``push``; returns at once (a ``concurrent.futures.Future`` carries completion)."""
        return self._pool().submit(self.push, key, t)

    def pull_async(self, key):
        return self._pool().submit(self.pull, key)

    def update_gradient_async(self, key, grad, version):
        return self._pool().submit(self.update_gradient, key, grad, version)

    def _pool(self):
        if getattr(self, "_executor", None) is None:
            from concurrent.futures import ThreadPoolExecutor
            self._executor = ThreadPoolExecutor(max_workers=2, thread_name_prefix="tfb-ps")
        return self._executor

    def barrier(self, ctx: Optional["DistributedContext"] = None):
        """Wait until queued work of this store is applied (and, with ``ctx``, until every rank got here)."""
        self.flush()
        if ctx is not None:
            ctx.barrier()

    def shutdown(self):
        self.stop()
        if getattr(self, "_executor", None) is not None:
            self._executor.shutdown(wait=True)
            self._executor = None

    def stop(self):
        self._stop = True
        if self._worker:
            self._worker.join(timeout=2)
