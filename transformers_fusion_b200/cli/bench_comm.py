"""``quant_bench --comm``: every fused compute + collective kernel against its library (NCCL + plain kernel) form.

Run under ``python -m torch.distributed.run --nproc-per-node N`` (one rank per GPU, all ranks one group).  Each line
gives, for one operation at one size: microseconds per call of the fused kernel and of the library form (CUDA events
around ``--iters`` back-to-back calls after warm-up, maximum over ranks), the bytes one rank moves over NVLink, the
resulting GB/s, and that as a fraction of ``--link-gbs`` (measured peer-copy bandwidth per direction).  For the GEMM
forms the roofline time is the slower of FLOPs / ``--gemm-tflops`` and NVLink bytes / link bandwidth.

Operations: zero2_step (reduce-scatter + AdamW + all-gather of a flat buffer), fsdp_reduce_scatter, all_reduce (one-shot /
two-shot sizes), ag_gemm (all-gather -> GEMM), gemm_rs (GEMM -> reduce-scatter), wg_gemm (weight gather -> GEMM)."""
from __future__ import annotations

import ctypes as C
import json
import os


def _timed(fn, iters, warmup, dist, dev):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms) * 1e3      # microseconds


def comm_bench(a):
    import torch
    import torch.distributed as dist

    from ..ops import _lib, functional as F
    from ..parallel.collectives import SymmCollectives
    from ..parallel.symm import SymmetricHeap
    from ..parallel.tp import TpContext, WeightGather, fused_gemm
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    assert world > 1, "run under torch.distributed.run with at least 2 ranks"
    heap = SymmetricHeap(rank, world, dev)
    W = world
    link, peak = a.link_gbs, a.gemm_tflops
    bf = torch.bfloat16
    it, wu = a.iters, a.warmup
    recs = []
    ops_wanted = set(getattr(a, "comm_ops", "all").split(","))
    on = lambda name: "all" in ops_wanted or name in ops_wanted

    def emit(op, size, us_f, us_l, nvl_bytes, flops=0.0):
        rec = {"op": op, "size": size, "world": W, "us_fused": round(us_f, 1), "us_library": round(us_l, 1),
               "speedup": round(us_l / us_f, 3), "nvlink_mb_per_rank": round(nvl_bytes / 1e6, 2),
               "fused_gbs": round(nvl_bytes / us_f / 1e3, 1), "frac_link_of_measured": round(nvl_bytes / us_f / 1e3 / link, 3)}
        if flops:
            roof = max(flops / (peak * 1e6), nvl_bytes / (link * 1e3))        # microseconds
            rec["tflops_fused"] = round(flops / us_f / 1e6, 1)
            rec["frac_roofline"] = round(roof / us_f, 3)
        recs.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    # ---------------------------------------------------------------- ZeRO-2 step on a flat buffer
    if on("zero2"):
        from ..models.dense import FlatBuffers
        from ..parallel.zero_fused import FusedZero
        from ..trainer.fused_optim import FlatAdamW

        class _Holder(torch.nn.Module):
            def __init__(self, n):
                super().__init__()
                self.w = torch.nn.Parameter(torch.zeros(n, dtype=bf, device=dev))
        n = a.zero_mb * (1 << 20) // 4 // (W * 1024) * (W * 1024)
        flat = FlatBuffers(_Holder(n), dtype=bf, pad_to=W * 1024, allocator=heap.alloc)
        per = flat.numel // W
        opt = FlatAdamW(flat, shard=(rank * per, (rank + 1) * per), norm_reduce=lambda t: dist.all_reduce(t))
        fz = FusedZero(flat, opt, heap, rank, W)
        opt.stage_hyper(None)

        def fused_zero():
            flat.grads.fill_(1e-3)
            fz.step()

        def lib_zero():
            flat.grads.fill_(1e-3)
            flat.grads.div_(W)
            lo, hi = rank * per, (rank + 1) * per
            dist.reduce_scatter_tensor(flat.grads[lo:hi], flat.grads)
            opt.step(staged=True)
            dist.all_gather_into_tensor(flat.params, flat.params[lo:hi].clone())
        nvl = (W - 1) * per * 4 + (W - 1) * per * 2           # peer loads of fp32 gradients + peer stores of bf16 parameters
        emit("zero2_step(rs+adamw+ag)", f"{flat.numel * 4 >> 20} MiB fp32 grads", _timed(fused_zero, it, wu, dist, dev),
             _timed(lib_zero, it, wu, dist, dev), nvl)
        del fz, opt, flat

    # ---------------------------------------------------------------- FSDP per-unit reduce-scatter
    if on("fsdp"):
        lib = _lib.lib()
        from ..parallel.sharded import _RsDesc
        lib.tfb_fsdp_reduce_scatter.argtypes = [C.POINTER(_RsDesc), C.c_int, C.c_void_p]
        lib.tfb_fsdp_reduce_scatter.restype = C.c_int
        nfull = a.unit_mb * (1 << 20) // 4 // (W * 512) * (W * 512)
        full = heap.alloc(nfull, torch.float32)
        fullv = full.view(torch.float32, nfull)
        fullv.fill_(1e-3)
        gshard = torch.zeros(nfull // W, dtype=torch.float32, device=dev)
        sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        ticket = torch.zeros(4, dtype=torch.int32, device=dev)
        d = _RsDesc()
        d.flag_ptrs, d.epoch, d.rank, d.world = heap.flags.ptrs.data_ptr(), heap.epoch.data_ptr(), rank, W
        d.status = _lib.status_word(dev).data_ptr()
        d.grad_ptrs, d.gshard, d.sumsq, d.ticket = full.ptrs.data_ptr(), gshard.data_ptr(), sumsq.data_ptr(), ticket.data_ptr()
        d.scale, d.nseg = 1.0 / W, 1
        d.seg[0], d.seg[1], d.seg[2] = 0, 0, nfull // W
        for ctas in (0, 148):
            us_f = _timed(lambda: _lib.check(lib.tfb_fsdp_reduce_scatter(C.byref(d), ctas, _lib.stream()), "fsdp_rs"), it, wu, dist, dev)
            us_l = _timed(lambda: dist.reduce_scatter_tensor(gshard, fullv, op=dist.ReduceOp.AVG), it, wu, dist, dev)
            emit(f"fsdp_reduce_scatter(ctas={ctas or 'all'})", f"{nfull * 4 >> 20} MiB fp32", us_f, us_l, (W - 1) * (nfull // W) * 4)

    # ---------------------------------------------------------------- FSDP per-unit weight all-gather (prefetch kernel)
    if on("fsdp"):
        from ..parallel.sharded import _AgDesc
        lib.tfb_fsdp_all_gather.argtypes = [C.POINTER(_AgDesc), C.c_int, C.c_void_p]
        lib.tfb_fsdp_all_gather.restype = C.c_int
        nsh = a.unit_mb * (1 << 20) // 2 // W // 512 * 512           # bf16 elements per shard
        shard = heap.alloc(nsh, bf)
        shard.view(bf, nsh).fill_(float(rank + 1))
        gathered = torch.zeros(nsh * W, dtype=bf, device=dev)
        srcs = torch.tensor(list(shard.peer_ptrs), dtype=torch.int64, device=dev)
        ad = _AgDesc()
        ad.rank, ad.world, ad.nseg = rank, W, 1
        ad.seg[0], ad.seg[1], ad.seg[2] = srcs.data_ptr(), gathered.data_ptr(), nsh * 2
        heap.barrier()
        us_f = _timed(lambda: _lib.check(lib.tfb_fsdp_all_gather(C.byref(ad), 0, _lib.stream()), "fsdp_ag"), it, wu, dist, dev)
        us_l = _timed(lambda: dist.all_gather_into_tensor(gathered, shard.view(bf, nsh)), it, wu, dist, dev)
        _lib.check(lib.tfb_fsdp_all_gather(C.byref(ad), 0, _lib.stream()), "fsdp_ag")
        torch.cuda.synchronize()
        want = torch.arange(1, W + 1, device=dev, dtype=torch.float32).repeat_interleave(nsh)
        assert torch.equal(gathered.float(), want), "fsdp_all_gather produced a wrong buffer"
        emit("fsdp_all_gather", f"{nsh * W * 2 >> 20} MiB bf16", us_f, us_l, (W - 1) * nsh * 2)

    # ---------------------------------------------------------------- small all-reduces
    if on("all_reduce"):
        sc = SymmCollectives(heap, capacity_bytes=64 << 20)
        for nbytes in (64 << 10, 256 << 10, 8 << 20, 64 << 20):
            t = torch.ones(nbytes // 2, dtype=bf, device=dev)
            u = t.clone()
            us_f = _timed(lambda: sc.all_reduce(t, "sum"), it, wu, dist, dev)
            us_l = _timed(lambda: dist.all_reduce(u), it, wu, dist, dev)
            one = nbytes <= sc.one_shot_max_bytes
            nvl = (W - 1) * nbytes if one else 2 * (W - 1) * nbytes // W
            emit("all_reduce(" + ("one-shot" if one else "two-shot") + ")", f"{nbytes >> 10} KiB bf16", us_f, us_l, nvl)
            t.fill_(1.0)
        # the decode form: a small local tensor, the residual stream added inside the kernel, sixteen calls replayed from a
        # CUDA graph like the layers of a decode step.  Library arm: NCCL all-reduce + add, launched eagerly back to back.
        for nbytes in (8 << 10, 64 << 10, 256 << 10):
            n = nbytes // 2
            res = torch.ones(n, dtype=bf, device=dev)
            xin = torch.ones(n, dtype=bf, device=dev)
            u = torch.ones(n, dtype=bf, device=dev)
            reps = 16

            def ll():
                for _ in range(reps):
                    sc.all_reduce_ll(xin, residual=res)

            def staged():
                for _ in range(reps):
                    sc.stage_view(bf, n)
                    sc.all_reduce_staged(n, bf, residual=res)

            def library():
                for _ in range(reps):
                    dist.all_reduce(u)
                    torch.add(u, res)
            side = torch.cuda.Stream(device=dev)
            us = []
            for fn in (ll, staged):
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    fn()
                torch.cuda.current_stream(dev).wait_stream(side)
                torch.cuda.synchronize()
                dist.barrier()
                g_ = torch.cuda.CUDAGraph()
                tok = sc.capture_begin()
                with torch.cuda.graph(g_):
                    fn()
                    sc.capture_end(tok)

                def replay():
                    sc.before_replay(tok)
                    g_.replay()
                us.append(_timed(replay, it, wu, dist, dev) / reps)
                torch.cuda.synchronize()
                g_.reset()
            us_l = _timed(library, it, wu, dist, dev) / reps
            u.fill_(1.0)
            emit("all_reduce+residual(flag-in-data, graph)", f"{nbytes >> 10} KiB bf16", us[0], us_l, (W - 1) * nbytes * 2)
            emit("all_reduce+residual(staged one-shot, graph)", f"{nbytes >> 10} KiB bf16", us[1], us_l, (W - 1) * nbytes)

    # ---------------------------------------------------------------- tensor-parallel GEMM pairs and the weight gather
    if on("tp_gemm"):
        M, H = a.tokens, a.hidden
        Nl = a.ffn // W * 2                                   # gate|up columns of one rank
        ctx = TpContext(heap, rank, W, M, H, H, copy_ctas=a.copy_ctas)
        g = torch.Generator(device=dev).manual_seed(rank)
        x_shard = (torch.randn(M // W, H, device=dev, generator=g)).to(bf)
        w_col = (torch.randn(Nl, H, device=dev, generator=g) * 0.02).to(bf)
        xs = [torch.empty_like(x_shard) for _ in range(W)]

        def lib_ag_gemm():
            xg = torch.empty((M, H), dtype=bf, device=dev)
            dist.all_gather_into_tensor(xg, x_shard)
            return F.gemm(xg, w_col)
        us_f = _timed(lambda: ctx.all_gather_gemm(x_shard, w_col), it, wu, dist, dev)
        us_l = _timed(lib_ag_gemm, it, wu, dist, dev)
        emit("ag_gemm", f"M{M} K{H} N{Nl}", us_f, us_l, (W - 1) * (M // W) * H * 2, 2.0 * M * H * Nl)
        Kl = a.ffn // W
        x_row = (torch.randn(M, Kl, device=dev, generator=g)).to(bf)
        w_row = (torch.randn(H, Kl, device=dev, generator=g) * 0.02).to(bf)

        def lib_gemm_rs():
            y = F.gemm(x_row, w_row)
            out = torch.empty((M // W, H), dtype=bf, device=dev)
            dist.reduce_scatter_tensor(out, y)
            return out
        us_f = _timed(lambda: ctx.gemm_reduce_scatter(x_row, w_row), it, wu, dist, dev)
        us_l = _timed(lib_gemm_rs, it, wu, dist, dev)
        emit("gemm_rs", f"M{M} K{Kl} N{H}", us_f, us_l, (W - 1) * (M // W) * H * 2, 2.0 * M * H * Kl)
        del ctx
        # weight gather -> GEMM: the [N, K] weight is row-sharded over the ranks
        N = a.ffn // 2 // (128 * W) * (128 * W)
        wsh = heap.alloc(N // W * H, bf)
        wsh.view(bf, N // W * H).copy_((torch.randn(N // W * H, device=dev, generator=g) * 0.02).to(bf))
        src = torch.tensor(wsh.peer_ptrs, dtype=torch.int64, device=dev)
        buf = torch.zeros((N, H), dtype=bf, device=dev)
        ready = torch.zeros(N // 128, dtype=torch.int32, device=dev)
        xfull = (torch.randn(M, H, device=dev, generator=g)).to(bf)
        ep = [0]

        wloc = wsh.view(bf, N // W * H).view(N // W, H)

        def f_wg():
            ep[0] += 1
            buf[rank * (N // W):(rank + 1) * (N // W)].copy_(wloc)          # own rows at HBM speed; the GEMM pulls the peers' rows
            return fused_gemm(xfull, buf, wg=WeightGather(buf, src, ready, ep[0], rank, W, skip_local=True), copy_ctas=a.copy_ctas)

        def l_wg():
            dist.all_gather_into_tensor(buf.view(-1), wsh.view(bf, N // W * H))
            return F.gemm(xfull, buf)
        us_f = _timed(f_wg, it, wu, dist, dev)
        us_l = _timed(l_wg, it, wu, dist, dev)
        emit("wg_gemm", f"M{M} K{H} N{N}", us_f, us_l, (W - 1) * (N // W) * H * 2, 2.0 * M * H * N)
        # the same gathered weight used with its rows as the reduction dimension (data-gradient product): every output tile
        # needs every row block, so the product can only finish once the whole gather has landed
        dy = (torch.randn(M, N, device=dev, generator=g)).to(bf)

        def f_wg_k():
            ep[0] += 1
            buf[rank * (N // W):(rank + 1) * (N // W)].copy_(wloc)
            return fused_gemm(dy, buf, b_mn=True, wg=WeightGather(buf, src, ready, ep[0], rank, W, skip_local=True), copy_ctas=a.copy_ctas)

        def l_wg_k():
            dist.all_gather_into_tensor(buf.view(-1), wsh.view(bf, N // W * H))
            return F.gemm(dy, buf, b_mn=True)
        us_f = _timed(f_wg_k, it, wu, dist, dev)
        us_l = _timed(l_wg_k, it, wu, dist, dev)
        emit("wg_gemm_dgrad", f"M{M} K{N} N{H}", us_f, us_l, (W - 1) * (N // W) * H * 2, 2.0 * M * H * N)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    dist.barrier()
    heap.close()
    dist.destroy_process_group()
    return recs
