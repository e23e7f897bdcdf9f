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
        torch.cuda.synchronize()
        res["status"] = int(_lib.status_word(dev)[0].item())
    json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    ctx.barrier()
    if symm is not None:
        symm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
