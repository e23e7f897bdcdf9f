"""Process-group mesh and the parallel training loops the command-line tools use.

One process per GPU, started by ``python -m torch.distributed.run``.  The world is factored as pp x dp x tp with tp
fastest (tensor-parallel peers exchange the most data per step), then dp, then pp:

    rank = (pp_idx * dp + dp_idx) * tp + tp_idx

``init_parallel`` builds the groups; ``fit_parallel`` runs the training loop that matches the factors:
  tp > 1 or zero stage 3   ShardedEngine: ZeRO-3 over the dp ranks x tensor + sequence parallelism over the tp ranks
                  (weight gather, all-gather->GEMM and GEMM->reduce-scatter inside the GEMM launches; symmetric heaps per
                  dp group and per tp group).  Model shapes it does not cover fall back to TPDenseModel + TPTrainer.
  ep > 1          MoE model with the experts of every layer spread over groups of ep ranks (fused dispatch / combine; ep < world: replicas), EPTrainer
  pp > 1          PipelineParallel 1F1B over the layer ranges, AdamW on the parameters each stage owns
  otherwise       the ordinary Trainer: data parallel with ZeRO stage 0 / 1 / 2 (fused reduce-scatter + AdamW)

Reference counterparts: DistributedContext (src/trainer/distributed.cpp:21-123), FSDP / DDP / pipeline /
tensor-parallel managers each taking a world size and a rank (src/trainer/{fsdp,ddp,pipeline,tensor_parallelism}.cpp);
the reference has no launcher that composes them."""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    rank: int = 0
    world: int = 1
    local_rank: int = 0
    device: torch.device = torch.device("cpu")
    dp: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    dp_rank: int = 0
    tp_rank: int = 0
    pp_rank: int = 0
    dp_group: object = None
    tp_group: object = None
    pp_group: object = None
    pp_ranks: Optional[List[int]] = None

    @property
    def is_main(self) -> bool:
        return self.rank == 0


def mesh_coords(rank: int, dp: int, tp: int, pp: int):
    """(pp_idx, dp_idx, tp_idx) of a rank."""
    return rank // (dp * tp), (rank // tp) % dp, rank % tp


def mesh_groups(world: int, dp: int, tp: int, pp: int):
    """Rank lists of every tp / dp / pp group, in the order all ranks must create them."""
    assert dp * tp * pp == world, f"dp x tp x pp = {dp * tp * pp} does not match the world size {world}"
    rk = lambda p, d, t: (p * dp + d) * tp + t
    tpg = [[rk(p, d, t) for t in range(tp)] for p in range(pp) for d in range(dp)]
    dpg = [[rk(p, d, t) for d in range(dp)] for p in range(pp) for t in range(tp)]
    ppg = [[rk(p, d, t) for p in range(pp)] for d in range(dp) for t in range(tp)]
    return tpg, dpg, ppg


def init_parallel(dp: int = 0, tp: int = 1, pp: int = 1, ep: int = 1, device: str = "auto", timeout_s: float = 600.0) -> ParallelState:
    """Joins the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT (a single process when they
    are unset) and builds the mesh groups.  ``dp = 0`` means "whatever is left of the world"."""
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() and device != "cpu"
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if dp <= 0:
        if world % (tp * pp):
            raise ValueError(f"world size {world} does not divide by tp x pp = {tp * pp}")
        dp = world // (tp * pp)
    if dp * tp * pp != world:
        raise ValueError(f"dp x tp x pp = {dp * tp * pp} does not match the world size {world}")
    if ep > 1 and (dp * tp) % ep:
        raise ValueError(f"the expert-parallel degree {ep} must divide dp x tp = {dp * tp}")
    st = ParallelState(rank, world, local, dev, dp, tp, pp, ep)
    st.pp_rank, st.dp_rank, st.tp_rank = mesh_coords(rank, dp, tp, pp)
    if world == 1:
        return st
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if use_cuda:
            torch.cuda.set_device(dev)
        kw = dict(device_id=dev) if use_cuda else {}
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    tpg, dpg, ppg = mesh_groups(world, dp, tp, pp)
    for ranks in tpg:
        g = dist.new_group(ranks) if tp > 1 else None
        if rank in ranks:
            st.tp_group = g
    for ranks in dpg:
        g = dist.new_group(ranks) if dp > 1 and dp < world else None
        if rank in ranks:
            st.dp_group = g                      # None = the default (whole-world) group when dp == world
    for ranks in ppg:
        g = dist.new_group(ranks) if pp > 1 else None
        if rank in ranks:
            st.pp_group, st.pp_ranks = g, ranks
    return st


def shutdown(st: ParallelState):
    if st.world > 1 and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------- training loops
def fit_parallel(model, tok, data_path: str, cfg, st: ParallelState, log: Optional[Callable] = None, resume: bool = False):
    """Runs ``cfg.max_steps`` (at most ``cfg.epochs`` passes) with the strategy the mesh asks for; rank 0 (for pp: the
    ranks that hold the pieces) writes ``cfg.checkpoint_path``.  Returns the last mean loss."""
    from ..trainer.trainer import DataLoader, Trainer
    from ..trainer.schedulers import schedule_lr
    dl = DataLoader(tok, data_path, cfg.batch_size, cfg.seq_length, device=st.device, rank=st.dp_rank, world=st.dp)
    steps = min(cfg.max_steps, max(1, len(dl)) * cfg.epochs)
    lr_at = lambda s: schedule_lr(cfg.lr_schedule, cfg.learning_rate, s, steps, min(cfg.warmup_steps, steps // 2))

    def report(step, loss, lr, toks, t0):
        import math
        import time
        if log and st.is_main and (step % max(1, cfg.log_interval) == 0 or step == steps):
            log(step, loss, math.exp(min(loss, 20.0)), lr, toks / max(1e-9, time.perf_counter() - t0))

    import time
    t0, toks, loss = time.perf_counter(), 0, 0.0
    sharded_ok = _sharded_supported(model.cfg, st) and st.pp == 1 and st.ep == 1
    if sharded_ok and (st.tp > 1 or (getattr(cfg, "zero_stage", 0) >= 3 and st.world > 1)):
        # ZeRO-3 over the dp ranks composed with tensor + sequence parallelism over the tp ranks; symmetric heaps span
        # exactly the dp group and the tp group of this rank, so the fused kernels work on any dp x tp factoring
        from .sharded import Mesh, ShardedEngine
        dp_heap = tp_heap = None
        comm = "nccl"
        if st.device.type == "cuda" and os.environ.get("TFB_COMM", "fused") == "fused":
            from .symm import SymmetricHeap
            comm = "fused"
            if st.dp > 1:
                dp_heap = SymmetricHeap(st.dp_rank, st.dp, st.device, group=st.dp_group)
            if st.tp > 1:
                tp_heap = SymmetricHeap(st.tp_rank, st.tp, st.device, group=st.tp_group)
        mesh = Mesh(st.dp_rank, st.dp, st.tp_rank, st.tp, st.dp_group, st.tp_group, None)
        eng = ShardedEngine.from_dense(model, mesh, comm=comm, dp_heap=dp_heap, tp_heap=tp_heap, lr=cfg.learning_rate,
                                       weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm,
                                       max_tokens=cfg.batch_size * cfg.seq_length)
        for step in range(1, steps + 1):
            ids, labels = dl.next_batch()
            lt = eng.train_step(ids, labels, lr_at(step)).detach().float().reshape(1).clone()
            if st.dp > 1:
                dist.all_reduce(lt, group=st.dp_group)
            loss = float(lt) / st.dp
            toks += ids.numel() * st.dp
            report(step, loss, lr_at(step), toks, t0)
        eng.export_to(model)
        if st.is_main:
            Trainer(model, tok).compile("adamw", _single(cfg)).save_checkpoint(cfg.checkpoint_path)
        return loss
    if st.tp > 1:
        # model shapes the sharded engine does not cover (LayerNorm, biases, learned positions): autograd-level tensor
        # parallelism with library collectives, gradients averaged over dp
        from .tp_model import TPDenseModel, TPGroup, TPTrainer
        ctx = None
        if st.device.type == "cuda" and os.environ.get("TFB_COMM", "fused") == "fused":
            from .symm import SymmetricHeap
            from .tp import TpContext
            c = model.cfg
            T = cfg.batch_size * cfg.seq_length
            widest = max(c.hidden_size, 2 * c.ffn_hidden_size // st.tp, (c.num_heads + 2 * c.num_kv_heads) * c.head_dim // st.tp)
            ctx = TpContext(SymmetricHeap(st.tp_rank, st.tp, st.device, group=st.tp_group), st.tp_rank, st.tp, T, widest, widest,
                            copy_ctas=8)
        tpm = TPDenseModel(model, TPGroup(st.tp_rank, st.tp, st.tp_group, ctx))
        tr = TPTrainer(tpm, cfg.learning_rate, cfg.weight_decay, cfg.max_grad_norm, st.dp_group if st.dp > 1 else None)
        for step in range(1, steps + 1):
            ids, labels = dl.next_batch()
            loss = tr.train_step(ids, labels, lr_at(step))
            toks += ids.numel() * st.dp
            report(step, loss, lr_at(step), toks, t0)
        tpm.gather_into(model)
        if st.is_main:
            Trainer(model, tok).compile("adamw", _single(cfg)).save_checkpoint(cfg.checkpoint_path)
        return loss
    if st.ep > 1:
        # expert parallel: every rank is a data-parallel rank of the replicated tensors; the experts of a layer are spread
        # over groups of `ep` consecutive ranks, and with ep < world every expert has world / ep replicas whose gradients
        # are summed over the ranks that hold the same experts
        if st.world % st.ep or st.tp > 1 or st.pp > 1 or not hasattr(model.cfg, "num_experts") or st.device.type != "cuda":
            raise ValueError("--ep needs a mixture-of-experts model on CUDA, tp = pp = 1 and ep dividing the number of ranks")
        from .ep_model import EPTrainer, attach_expert_parallel
        from .symm import SymmetricHeap
        ep_rank, replicas = st.rank % st.ep, st.world // st.ep
        ep_group = replica_group = None
        if replicas > 1:
            for g in range(replicas):
                grp = dist.new_group(list(range(g * st.ep, (g + 1) * st.ep)))
                if st.rank // st.ep == g:
                    ep_group = grp
            for e in range(st.ep):
                grp = dist.new_group([e + g * st.ep for g in range(replicas)])
                if ep_rank == e:
                    replica_group = grp
        symm = SymmetricHeap(ep_rank, st.ep, st.device, group=ep_group)
        experts = attach_expert_parallel(model, symm, ep_rank, st.ep, cfg.batch_size * cfg.seq_length)
        tr = EPTrainer(model, experts, cfg.learning_rate, cfg.weight_decay, cfg.max_grad_norm, replica_group=replica_group,
                       replicas=replicas)
        for step in range(1, steps + 1):
            ids, labels = dl.next_batch()
            loss = tr.train_step(ids, labels, lr_at(step))
            toks += ids.numel() * st.world
            report(step, loss, lr_at(step), toks, t0)
        return loss
    if st.pp > 1:
        from ..engines.dense import OptimSuite
        from .collectives import DistributedContext
        from .pp import PipelineParallel
        pipe = PipelineParallel(model, st.pp, st.pp_rank, DistributedContext(st.pp_rank, st.pp, st.pp_group),
                                num_microbatches=min(4, cfg.batch_size), stage_ranks=st.pp_ranks)
        opt = OptimSuite("adamw", cfg.learning_rate, cfg.weight_decay)
        owned = pipe.owned_parameters()
        opt.add_group(owned, 1.0, 1.0)
        last_rank = st.pp_ranks[-1]
        for step in range(1, steps + 1):
            ids, labels = dl.next_batch()
            l = pipe.run_1f1b(ids, labels)
            lt = torch.zeros(1, device=st.device) if l is None else l.detach().reshape(1).float()
            dist.broadcast(lt, last_rank, group=st.pp_group)
            if st.dp > 1:
                for p in owned:
                    dist.all_reduce(p.main_grad, group=st.dp_group)
                    p.main_grad.div_(st.dp)
            opt.set_lr(lr_at(step))
            pipe.clip_gradients(cfg.max_grad_norm)      # global norm over every stage; a tied embedding counted once
            opt.step()
            pipe.clear_accumulated_gradients()
            loss = float(lt)
            toks += ids.numel() * st.dp
            report(step, loss, lr_at(step), toks, t0)
        # every stage sends its owned tensors to rank 0 of its pipeline, which then holds the full model
        _collect_pipeline(model, pipe, st)
        if st.is_main:
            Trainer(model, tok).compile("adamw", _single(cfg)).save_checkpoint(cfg.checkpoint_path)
        return loss
    if getattr(cfg, "zero_stage", 0) >= 3 and st.world > 1:
        raise ValueError("--zero-stage 3 covers RoPE + RMSNorm models without biases; use --zero-stage 2 for this model")
    tr = Trainer(model, tok).compile(None, cfg)
    if log:
        tr.set_log_callback(lambda m: st.is_main and log(m.step, m.loss, m.perplexity, m.learning_rate, m.tokens_per_sec * st.dp))
    if resume and os.path.exists(cfg.checkpoint_path):
        tr.load_checkpoint(cfg.checkpoint_path, dl)
    if not st.is_main:
        tr.cfg.save_interval = 1 << 60                 # only rank 0 writes checkpoints
    tr.fit(dl)
    return tr.metrics().loss


def _sharded_supported(c, st) -> bool:
    """Model shapes parallel.sharded.ShardedEngine covers on this mesh."""
    return (getattr(c, "norm_type", "") == "rmsnorm" and not c.use_parallel_residual and not c.attention_bias and
            c.position_type == "rope" and not hasattr(c, "num_experts") and c.num_heads % st.tp == 0 and
            c.num_kv_heads % st.tp == 0 and c.ffn_hidden_size % st.tp == 0 and c.vocab_size % st.tp == 0 and
            getattr(c, "mtp_num_heads", 0) == 0)


def _single(cfg):
    import copy
    c = copy.copy(cfg)
    c.zero_stage = 0
    return c


@torch.no_grad()
def _collect_pipeline(model, pipe, st: ParallelState):
    """Broadcast every stage's owned tensors inside its pipeline group so that all stages end with the full model."""
    from .pp import split_model
    for s in range(st.pp):
        lo, hi = split_model(model.cfg.num_layers, st.pp, pipe.balance)[s]
        ts = [p.data for i in range(lo, hi) for p in model.layers[i].parameters()]
        if s == 0:
            ts.append(model.tok_embeddings.data)
        if s == st.pp - 1:
            ts.append(model.norm.data)
            if not (model.cfg.tie_embeddings):
                ts.append(model.lm_head.data)
        for t in ts:
            dist.broadcast(t, st.pp_ranks[s], group=st.pp_group)
