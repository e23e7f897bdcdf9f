"""FSDP worker.  argv: <out_dir> <backend>.  ZeRO-3 training must follow single-process AdamW training; with nccl the
weight gather runs inside the GEMM launches."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import TransformerConfig  # noqa: E402
from transformers_fusion_b200.models.dense import DenseModel  # noqa: E402
from transformers_fusion_b200.parallel.collectives import DistributedContext  # noqa: E402
from transformers_fusion_b200.parallel.fsdp import FSDPConfig, FullyShardedDataParallel  # noqa: E402


def main():
    out_dir, backend = sys.argv[1], sys.argv[2]
    ctx = DistributedContext.init(backend)
    rank, world = ctx.rank, ctx.world_size
    gpu = backend == "nccl"
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"])) if gpu else torch.device("cpu")
    dt = torch.bfloat16 if gpu else torch.float32
    H = 256 if gpu else 256
    cfg = TransformerConfig(vocab_size=512, hidden_size=H, num_layers=2, num_heads=4, ffn_hidden_size=512, max_seq_len=128)
    symm = None
    if gpu:
        from transformers_fusion_b200.ops import _lib
        from transformers_fusion_b200.parallel.symm import SymmetricHeap
        symm = SymmetricHeap(rank, world, dev)
    S = 128 if gpu else 16
    g = torch.Generator().manual_seed(0)
    ids_all = torch.randint(0, 512, (2 * world, S), generator=g)
    lab_all = torch.roll(ids_all, -1, 1)
    # reference: one process, whole batch, same AdamW
    ref = DenseModel(cfg, device=dev, dtype=dt, seed=3)
    ref_f = FullyShardedDataParallel(ref, FSDPConfig(lr=1e-2, weight_decay=0.0), DistributedContext(0, 1))
    ref_f.engine.mesh.world_group = None
    m = DenseModel(cfg, device=dev, dtype=dt, seed=3)
    fs = FullyShardedDataParallel(m, FSDPConfig(lr=1e-2, weight_decay=0.0, copy_ctas=4), ctx, symm)
    res = {"n_sharded": len(fs.weights), "savings": fs.memory_savings_ratio()}
    losses, ref_losses = [], []
    for step in range(3):
        fs.scrub()                                  # peers' rows are gone: every use must gather them again
        mine = slice(2 * rank, 2 * rank + 2)
        loss = fs.train_step(ids_all[mine].to(dev), lab_all[mine].to(dev))
        lt = torch.tensor([float(loss)], device=dev)
        ctx.all_reduce(lt, "avg")
        losses.append(float(lt))
        ref_losses.append(float(ref_f.train_step(ids_all.to(dev), lab_all.to(dev))))
    res["losses"], res["ref_losses"] = losses, ref_losses
    fs.consolidate()
    ref_f.consolidate()
    err = 0.0
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        err = max(err, float((p.data.float() - q.data.float()).abs().max()))
    res["param_err"] = err
    res["gathers"] = fs.gathers
    if gpu:
        torch.cuda.synchronize()
        res["status"] = int(_lib.status_word(dev)[0].item())
    json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    ctx.barrier()
    if symm is not None:
        symm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
