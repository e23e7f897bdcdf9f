"""Worker for the tensor-parallel tests (one rank per device): fused all-gather->GEMM and
GEMM->reduce-scatter against the single-device product.  argv: <out_dir>."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.ops import _lib  # noqa: E402
from transformers_fusion_b200.parallel.symm import SymmetricHeap  # noqa: E402
from transformers_fusion_b200.parallel.tp import TpContext  # noqa: E402


def main():
    out_dir = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    symm = SymmetricHeap(rank, world, dev)
    M, K, N = 1024 * world, 512, 768
    ctx = TpContext(symm, rank, world, M, max(K, N), max(K, N), copy_ctas=8)
    g = torch.Generator().manual_seed(5)
    X = torch.randn(M, K, generator=g).bfloat16()
    Wc = torch.randn(N, K, generator=g).bfloat16()       # column-parallel weight (full)
    Wr = torch.randn(K, N, generator=g).bfloat16()       # row-parallel weight (full): [out=K, in=N]
    res = {}
    Ms, Nl = M // world, N // world
    for rep in range(3):   # repeated calls exercise the double buffering and the epoch logic
        x_shard = X[rank * Ms:(rank + 1) * Ms].to(dev)
        w_local = Wc[rank * Nl:(rank + 1) * Nl].to(dev)
        y, _ = ctx.all_gather_gemm(x_shard, w_local)
        ref = (X.float() @ Wc[rank * Nl:(rank + 1) * Nl].float().t())
        res[f"ag_gemm_err_{rep}"] = (y.float().cpu() - ref).abs().max().item() / ref.abs().max().item()
        # row parallel: input y-like activation [M, N/W] local slice of the hidden dim
        A = torch.randn(M, N, generator=torch.Generator().manual_seed(9 + rep)).bfloat16()
        a_local = A[:, rank * Nl:(rank + 1) * Nl].contiguous().to(dev)
        wr_local = Wr[:, rank * Nl:(rank + 1) * Nl].contiguous().to(dev)
        resid = torch.randn(Ms, K, generator=torch.Generator().manual_seed(20 + rank)).bfloat16().to(dev)
        z = ctx.gemm_reduce_scatter(a_local, wr_local, resid)
        full = A.float() @ Wr.float().t()
        refz = full[rank * Ms:(rank + 1) * Ms] + resid.float().cpu()
        res[f"gemm_rs_err_{rep}"] = (z.float().cpu() - refz).abs().max().item() / refz.abs().max().item()
    torch.cuda.synchronize()
    res["status"] = int(_lib.status_word(dev)[0].item())
    json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    dist.barrier()
    symm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
