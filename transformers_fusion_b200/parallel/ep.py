"""Expert parallelism: experts sharded across ranks (contiguous blocks, E / W per rank), tokens
exchanged by the fused dispatch / combine kernels over NVLink peer memory (csrc/comm/ep_fused.cu).

Forward on every rank:  route local tokens -> push the count row to all ranks -> plan (identical on all
ranks) -> dispatch (token rows stored straight into the owners' expert input buffers) -> grouped expert
GEMMs on the owner -> combine (weighted sum of rows read from the owners' output buffers).  Three flag
barriers separate the phases.  Backward mirrors it.  Non-expert gradients are reduced by data
parallelism as usual; expert weights live only on their owner, so their gradients need no reduction
(``expert_dp_group`` would average replicas when EP < world).

Reference counterparts: ExpertParallel (round-robin experts, replicated tokens + all-reduce combine,
src/model/moe_model.cpp:508-700), assign_experts_to_nodes contiguous blocks (src/model/expert_parallel.cpp:319),
ExpertDispatcher::route_tokens / plan_all_to_all (:354-555)."""
from __future__ import annotations

import torch

from ..ops import _lib, functional as F, moe as M
from ..ops._lib import c_i, c_p, check, stream

_lib.register("tfb_ep_push_counts", [c_p, c_p, c_i, c_i, c_i, c_p])
_lib.register("tfb_ep_plan", [c_p, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_p, c_p, c_p])
_lib.register("tfb_ep_dispatch", [c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p])
_lib.register("tfb_ep_combine", [c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p])
_lib.register("tfb_ep_combine_bwd", [c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p])
_lib.register("tfb_ep_dispatch_bwd", [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_p])


def assign_experts(num_experts: int, world: int):
    """Contiguous blocks: rank r owns experts [r * E/W, (r+1) * E/W)."""
    per = num_experts // world
    return [list(range(r * per, (r + 1) * per)) for r in range(world)]


class _EpPlan:
    pass


class ExpertParallel:
    def __init__(self, symm, rank, world, num_experts, hidden, max_tokens, top_k, capacity_factor=None, resident=False):
        """``resident``: this object serves ONE layer and every forward is followed by its backward before the next
        forward.  The dispatched rows and the expert outputs then stay in the symmetric buffers until the backward
        (no copies out and back), gradients arrive in a third buffer, and a layer crosses five flag barriers instead
        of eight.  A backward that finds the buffers overwritten by a later forward raises."""
        assert num_experts % world == 0
        self.symm, self.rank, self.world, self.E, self.H = symm, rank, world, num_experts, hidden
        self.El = num_experts // world
        cf = world if capacity_factor is None else capacity_factor
        self.max_rows = (int(cf * max_tokens * top_k) + 127) // 128 * 128 + 128 * self.El
        self.max_tiles = self.max_rows // 128
        dev = symm.device
        bf = torch.bfloat16
        self.xp = symm.alloc(self.max_rows * hidden, bf)     # dispatch target / dxp source
        self.yp = symm.alloc(self.max_rows * hidden, bf)     # combine source / dyp target
        self.counts_all = symm.alloc(world * num_experts, torch.int32)
        self.resident, self.generation = resident, 0
        self.gp = symm.alloc(self.max_rows * hidden, bf) if resident else None     # dyp target
        self.dev = dev

    def _t(self, buf, dtype=torch.bfloat16):
        return buf.view(dtype, self.max_rows * self.H).view(self.max_rows, self.H)

    def local_experts(self):
        return assign_experts(self.E, self.world)[self.rank]

    def num_experts(self) -> int: return self.E
    def num_local_experts(self) -> int: return self.El
    def num_ranks(self) -> int: return self.world

    def forward(self, x, logits, gate_up_local, down_local, k, renorm=True, act=0, lb_weight=0.0, z_weight=0.0):
        """``moe_ffn`` under the name the reference's wrappers use (include/quant/moe_enhance.h:94-98; the model-level
        wrapper with attach / forward_with_parallel / sync_gradients is ``parallel.ep_model.ModelExpertParallel``)."""
        return self.moe_ffn(x, logits, gate_up_local, down_local, k, renorm, act, lb_weight, z_weight)

    def moe_ffn(self, x, logits, gate_up_local, down_local, k, renorm, act, lb_weight, z_weight):
        """Same contract as ops.moe.moe_ffn, with gate_up_local / down_local holding only this rank's experts."""
        return _EpFFN.apply(x, logits, gate_up_local, down_local, self, k, renorm, act, lb_weight, z_weight)


class _EpFFN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, logits, gate_up, down, ep: ExpertParallel, k, renorm, act, lb_weight, z_weight):
        lib, s = _lib.lib(), stream
        T, H = x.shape
        E, El, W, rank, dev = ep.E, ep.El, ep.world, ep.rank, x.device
        idx, w, probs, counts, lse = M.router_topk(logits, k, renorm)
        xp, yp = ep._t(ep.xp), ep._t(ep.yp)
        xp.zero_()
        ep.generation += 1
        if ep.resident:
            ep._t(ep.gp).zero_()          # ordered before this forward's barriers, so peers' gradient rows land on zeros
        check(lib.tfb_ep_push_counts(counts.data_ptr(), ep.counts_all.ptrs.data_ptr(), W, E, rank, s()), "ep_push_counts")
        ep.symm.barrier()
        pl = _EpPlan()
        pl.base = torch.empty(E, dtype=torch.int32, device=dev)
        pl.cursor = torch.empty(E, dtype=torch.int32, device=dev)
        pl.seg_start = torch.empty(El + 1, dtype=torch.int32, device=dev)
        pl.expert_of_tile = torch.empty(ep.max_tiles, dtype=torch.int32, device=dev)
        pl.total = torch.empty(1, dtype=torch.int32, device=dev)
        pl.row_of = torch.empty((T, k), dtype=torch.int32, device=dev)
        pl.T, pl.k, pl.E, pl.max_rows, pl.max_tiles = T, k, El, ep.max_rows, ep.max_tiles
        ca = ep.counts_all.view(torch.int32, W * E)
        check(lib.tfb_ep_plan(ca.data_ptr(), W, E, rank, pl.base.data_ptr(), pl.seg_start.data_ptr(),
                              pl.expert_of_tile.data_ptr(), ep.max_tiles, pl.total.data_ptr(), pl.cursor.data_ptr(), s()),
              "ep_plan")
        check(lib.tfb_ep_dispatch(x.data_ptr(), idx.data_ptr(), pl.base.data_ptr(), pl.cursor.data_ptr(),
                                  pl.row_of.data_ptr(), ep.xp.ptrs.data_ptr(), T, k, H, El, ep.max_rows, s()), "ep_dispatch")
        # global token fractions for the load-balance loss; read before the barrier below so that no peer can
        # already be pushing the counts of its next layer
        f_glob = ca.view(W, E).float().sum(0)
        f_glob = f_glob / f_glob.sum().clamp(min=1)
        ep.symm.barrier()                              # every token row has reached its owner
        xp_saved = xp if ep.resident else xp.clone()
        gu = M.grouped_gemm(xp_saved, gate_up.data, pl)
        a = F.glu_fwd(gu, act, rows=pl.total)          # only the routed rows; the provisioned tail is never read
        M.grouped_gemm(a, down.data, pl, out=yp)        # straight into the buffer the sources read in combine
        ep.symm.barrier()                              # expert outputs are readable by the sources
        y = torch.empty((T, H), dtype=x.dtype, device=dev)
        check(lib.tfb_ep_combine(ep.yp.ptrs.data_ptr(), idx.data_ptr(), pl.row_of.data_ptr(), w.data_ptr(), y.data_ptr(),
                                 T, k, H, El, s()), "ep_combine")
        aux = lb_weight * E * (f_glob * probs.mean(0)).sum() + z_weight * (lse * lse).mean()
        if ep.resident:
            ctx.save_for_backward(x, gu, a, w, probs, idx, lse, f_glob)
        else:
            ctx.save_for_backward(x, gu, a, w, probs, idx, lse, f_glob, xp_saved, yp.clone())
        ctx.generation = ep.generation
        ctx.pl, ctx.ep, ctx.gate_up, ctx.down = pl, ep, gate_up, down
        ctx.cfg = (k, renorm, act, lb_weight, z_weight)
        ctx.logits_dtype = logits.dtype
        ctx.mark_non_differentiable(idx)
        return y, aux, idx

    @staticmethod
    def backward(ctx, dy, daux, _didx):
        lib, s = _lib.lib(), stream
        pl, ep, gate_up, down = ctx.pl, ctx.ep, ctx.gate_up, ctx.down
        if ep.resident:
            x, gu, a, w, probs, idx, lse, f_glob = ctx.saved_tensors
            if ctx.generation != ep.generation:
                raise RuntimeError("resident expert-parallel buffers were overwritten by a later forward; build "
                                   "ExpertParallel(resident=False) for schedules that run two forwards before a backward")
        else:
            x, gu, a, w, probs, idx, lse, f_glob, xp_saved, yp_saved = ctx.saved_tensors
        k, renorm, act, lb_weight, z_weight = ctx.cfg
        T, H = x.shape
        E, El = ep.E, ep.El
        dev = x.device
        dy = dy.contiguous()
        xp_sym, yp_sym = ep._t(ep.xp), ep._t(ep.yp)
        if ep.resident:
            xp_saved, grad_buf, dyp_sym = xp_sym, ep.gp, ep._t(ep.gp)      # outputs still exposed, gp cleared in forward
        else:
            yp_sym.copy_(yp_saved)                      # owners re-expose their outputs (needed for d weights)
            xp_sym.zero_()                              # xp buffer now receives dyp rows
            ep.symm.barrier()
            grad_buf, dyp_sym = ep.xp, xp_sym
        dw = torch.empty((T, k), dtype=torch.float32, device=dev)
        check(lib.tfb_ep_combine_bwd(dy.data_ptr(), ep.yp.ptrs.data_ptr(), grad_buf.ptrs.data_ptr(), idx.data_ptr(),
                                     pl.row_of.data_ptr(), w.data_ptr(), dw.data_ptr(), T, k, H, El, s()), "ep_combine_bwd")
        ep.symm.barrier()                               # gradient rows have reached the owners
        for p_ in (gate_up, down):
            if not hasattr(p_, "main_grad") or p_.main_grad is None:
                p_.main_grad = torch.zeros(p_.shape, dtype=torch.float32, device=dev)
        dyp = dyp_sym if ep.resident else dyp_sym.clone()
        da = M.grouped_gemm(dyp, down.data, pl, b_mn=True)
        M.grouped_wgrad(dyp, a, pl, down.main_grad)
        dgu = F.glu_bwd(gu, da, act, rows=pl.total)
        M.grouped_gemm(dgu, gate_up.data, pl, b_mn=True, out=yp_sym)     # dxp, exposed through the yp buffer
        M.grouped_wgrad(dgu, xp_saved, pl, gate_up.main_grad)
        ep.symm.barrier()                               # dxp rows are readable by the sources
        dx = torch.empty((T, H), dtype=x.dtype, device=dev)
        check(lib.tfb_ep_dispatch_bwd(ep.yp.ptrs.data_ptr(), idx.data_ptr(), pl.row_of.data_ptr(), dx.data_ptr(), T, k, H,
                                      El, s()), "ep_dispatch_bwd")
        if not ep.resident:                             # resident: the next writer of these buffers is this layer's next
            ep.symm.barrier()                           # forward, which crosses two barriers first
        # router gradient (local tokens): identical to the single-rank expression
        dprobs = torch.zeros_like(probs)
        li = idx.long()
        sel = probs.gather(1, li)
        if renorm:
            ssum = sel.sum(-1, keepdim=True)
            dsel = dw / ssum - (dw * sel).sum(-1, keepdim=True) / (ssum * ssum)
        else:
            dsel = dw
        dprobs.scatter_add_(1, li, dsel)
        daux = daux if daux is not None else torch.zeros((), device=dev)
        dprobs = dprobs + daux * lb_weight * E * f_glob[None, :] / T
        dlogits = probs * (dprobs - (dprobs * probs).sum(-1, keepdim=True))
        dlogits = dlogits + daux * z_weight * (2.0 / T) * lse[:, None] * probs
        return dx, dlogits.to(ctx.logits_dtype), None, None, None, None, None, None, None, None
