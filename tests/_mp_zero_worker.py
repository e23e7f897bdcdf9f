"""Worker for the multi-process ZeRO tests (launched by torch.distributed.run, one rank per device).
argv: <backend> <out_dir>.  Runs the same 3 optimizer steps with every gradient path available on the
backend and writes max-abs differences between the resulting parameters to <out_dir>/rank<r>.json."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import TransformerConfig  # noqa: E402
from transformers_fusion_b200.models.dense import DenseModel  # noqa: E402
from transformers_fusion_b200.trainer.engine import TrainEngine  # noqa: E402


def main():
    backend, out_dir = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = backend == "nccl"
    if cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
        dtype = torch.bfloat16
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype = torch.float32
    cfg = TransformerConfig(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                            ffn_hidden_size=512, max_seq_len=128, init_std=0.05, tie_embeddings=True)
    S, B = 128, 2
    g = torch.Generator().manual_seed(100)
    all_ids = torch.randint(0, cfg.vocab_size, (3, world * B, S), generator=g)

    def run(comm, zero_stage, graph=False):
        symm = None
        if comm == "fused":
            from transformers_fusion_b200.parallel.symm import SymmetricHeap
            symm = SymmetricHeap(rank, world, dev)
        model = DenseModel(cfg, device=dev, dtype=dtype, seed=11)
        eng = TrainEngine(model, lr=1e-2, weight_decay=0.1, max_grad_norm=0.5, zero_stage=zero_stage, comm=comm,
                          symm=symm, cuda_graph=graph)
        losses = []
        for step in range(3):
            ids = all_ids[step, rank * B:(rank + 1) * B].to(dev)
            losses.append(float(eng.step(ids, torch.roll(ids, -1, 1)).item()))
        if cuda:
            torch.cuda.synchronize()
            from transformers_fusion_b200.ops import _lib
            _lib.check_status(dev)
        out = eng.flat.params.float().cpu().clone(), losses, float(eng.opt.grad_norm.item())
        if symm is not None:
            del eng, model
            symm.close()
        return out

    res = {}
    base, base_l, base_n = run("nccl", 0)
    z2, z2_l, z2_n = run("nccl", 2)
    res["zero2_vs_ddp"] = (base - z2).abs().max().item()
    res["losses_ddp"], res["losses_zero2"] = base_l, z2_l
    res["norm_ddp"], res["norm_zero2"] = base_n, z2_n
    if cuda:
        fz, fz_l, fz_n = run("fused", 2)
        res["fused_vs_ddp"] = (base - fz).abs().max().item()
        res["losses_fused"], res["norm_fused"] = fz_l, fz_n
        fg, fg_l, _ = run("fused", 2, graph=True)
        res["fused_graph_vs_ddp"] = (base - fg).abs().max().item()
        res["losses_fused_graph"] = fg_l
    res["param_absmax"] = base.abs().max().item()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
