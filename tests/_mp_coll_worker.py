"""Worker for the collective tests.  argv: <out_dir> <backend: gloo|nccl>.  With nccl the fused symmetric-memory
kernels are checked against torch.distributed; with gloo only the host API runs."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.parallel.collectives import DistributedContext, RingAllReduce, SymmCollectives  # noqa: E402


def main():
    out_dir, backend = sys.argv[1], sys.argv[2]
    ctx = DistributedContext.init(backend)
    rank, world = ctx.rank, ctx.world_size
    res = {}
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"])) if backend == "nccl" else torch.device("cpu")
    sc = symm = None
    if backend == "nccl":
        from transformers_fusion_b200.ops import _lib
        from transformers_fusion_b200.parallel.symm import SymmetricHeap
        symm = SymmetricHeap(rank, world, dev)
        sc = SymmCollectives(symm, 4 << 20)
    ring = RingAllReduce(ctx, sc)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(1000, generator=g).to(dev)
    allx = [torch.randn(1000, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
    for op, ref in (("sum", sum(allx)), ("avg", sum(allx) / world), ("max", torch.stack(allx).amax(0)), ("min", torch.stack(allx).amin(0))):
        y = ring.allreduce(x.clone(), op)
        res[f"allreduce_{op}"] = (y.cpu() - ref).abs().max().item()
    res["chunked"] = (ring.allreduce_chunked(x.clone(), "sum", 300).cpu() - sum(allx)).abs().max().item()
    t = torch.arange(4 * world, dtype=torch.float32).view(2 * world, 2).to(dev) + rank
    rs = ring.reduce_scatter(t.clone())
    full = sum(torch.arange(4 * world, dtype=torch.float32).view(2 * world, 2) + r for r in range(world))
    res["reduce_scatter"] = (rs.cpu() - full[2 * rank:2 * rank + 2]).abs().max().item()
    ag = ring.allgather(torch.full((2, 3), float(rank), device=dev))
    res["allgather"] = float((ag.cpu() - torch.arange(world).float().repeat_interleave(2)[:, None]).abs().max())
    sc_t = ring.scatter(torch.arange(2 * world, dtype=torch.float32).to(dev) * (1 if rank == 0 else -1), root=0)
    res["scatter"] = float((sc_t.cpu() - torch.arange(2 * rank, 2 * rank + 2).float()).abs().max())
    b = ctx.broadcast(torch.full((5,), float(rank), device=dev), root=world - 1)
    res["broadcast"] = float((b.cpu() - (world - 1)).abs().max())
    if sc is not None:
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 5e-2)):
            for n in (8, 1000, 70000, 600000):
                xs = [torch.randn(n, generator=torch.Generator().manual_seed(7 * r + n)).to(dtype) for r in range(world)]
                ref = sum(v.float() for v in xs)
                for algo in ("one_shot", "two_shot"):
                    for rep in range(2):
                        y = sc.all_reduce(xs[rank].to(dev).clone(), "sum", algo)
                        res[f"sc_{algo}_{dtype}_{n}_{rep}"] = ((y.float().cpu() - ref).abs().max() / tol).item()
        xs = [torch.randn(4096 * world, generator=torch.Generator().manual_seed(r)) for r in range(world)]
        out = sc.reduce_scatter(xs[rank].to(dev), "avg")
        res["sc_reduce_scatter"] = (out.cpu() - (sum(xs) / world)[4096 * rank:4096 * (rank + 1)]).abs().max().item() / 1e-5
        ag = sc.all_gather(torch.full((2048,), float(rank + 1), device=dev, dtype=torch.bfloat16))
        res["sc_all_gather"] = float((ag.float().cpu() - torch.arange(1, world + 1).float().repeat_interleave(2048)).abs().max())
        bt = sc.broadcast(torch.full((777,), float(rank), device=dev), root=1)
        res["sc_broadcast"] = float((bt.cpu() - 1.0).abs().max())
        # staged all-reduce with the residual added inside the kernel; eager, then replayed from a graph that was
        # captured with an odd number of collectives, with eager collectives in between the replays
        n = 4096
        parts = [torch.randn(n, generator=torch.Generator().manual_seed(50 + r)).to(torch.bfloat16) for r in range(world)]
        resid = torch.randn(n, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
        ref = (sum(v.float() for v in parts) + resid.float())
        mine, rdev = parts[rank].to(dev), resid.to(dev)

        def staged_once():
            sc.stage_view(torch.bfloat16, n).copy_(mine)
            return sc.all_reduce_staged(n, torch.bfloat16, residual=rdev)
        res["sc_staged_residual"] = float((staged_once().float().cpu() - ref).abs().max() / 5e-2)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            staged_once()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        tok = sc.capture_begin()
        with torch.cuda.graph(graph):
            outs = [staged_once() for _ in range(3)]
            sc.capture_end(tok)
        worst = 0.0
        for rep in range(4):
            sc.before_replay(tok)
            graph.replay()
            worst = max(worst, max(float((o.float().cpu() - ref).abs().max()) for o in outs))
            if rep % 2 == 0:       # an odd number of eager collectives between two replays
                worst = max(worst, float((staged_once().float().cpu() - ref).abs().max()))
        res["sc_staged_graph"] = worst / 5e-2
        # flag-in-data all-reduce: every op and dtype eagerly, then (sum + residual, in place) replayed from a graph with
        # eager calls in between; sizes from one 16-byte vector to the largest message
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 5e-2)):
            for n_ll in (8, 4096, sc.one_shot_max_bytes // 4):
                xs = [torch.randn(n_ll, generator=torch.Generator().manual_seed(11 * r + n_ll)).to(dtype) for r in range(world)]
                st_ = torch.stack([v.float() for v in xs])
                for op, want in (("sum", st_.sum(0)), ("avg", st_.mean(0)), ("max", st_.amax(0)), ("min", st_.amin(0))):
                    for rep in range(2):
                        y = sc.all_reduce_ll(xs[rank].to(dev), op)
                        res[f"sc_ll_{op}_{dtype}_{n_ll}_{rep}"] = float((y.float().cpu() - want).abs().max() / tol)

        def ll_once():
            buf = mine.clone()
            return sc.all_reduce_ll(buf, residual=rdev, out=buf)
        res["sc_ll_residual"] = float((ll_once().float().cpu() - ref).abs().max() / 5e-2)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            ll_once()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2):
            outs2 = [ll_once() for _ in range(3)]
        worst = 0.0
        for rep in range(4):
            graph2.replay()
            worst = max(worst, max(float((o.float().cpu() - ref).abs().max()) for o in outs2))
            if rep % 2 == 0:
                worst = max(worst, float((ll_once().float().cpu() - ref).abs().max()))
        res["sc_ll_graph"] = worst / 5e-2
        torch.cuda.synchronize()
        res["status"] = int(_lib.status_word(dev)[0].item())
    json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    ctx.barrier()
    if symm is not None:
        symm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
