"""Worker for the expert-parallel model test: the EP model's loss on this rank's batch equals the loss of the full model
on the same batch, a few optimiser steps reduce the loss, replicated tensors stay identical across ranks.
argv: <out_dir>."""
import copy
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import MoEConfig  # noqa: E402
from transformers_fusion_b200.models.moe import MoEModel  # noqa: E402
from transformers_fusion_b200.ops import _lib  # noqa: E402
from transformers_fusion_b200.parallel.ep_model import EPTrainer, attach_expert_parallel  # noqa: E402
from transformers_fusion_b200.parallel.symm import SymmetricHeap  # noqa: E402


def main():
    out_dir = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    symm = SymmetricHeap(rank, world, dev)
    cfg = MoEConfig(vocab_size=256, hidden_size=128, num_layers=2, num_heads=2, ffn_hidden_size=256, max_seq_len=128, init_std=0.08,
                    num_experts=4, top_k=2, expert_hidden_size=128)
    full = MoEModel(cfg, device=dev, dtype=torch.bfloat16, seed=7)
    full.flatten()
    model = copy.deepcopy(full)
    model.flat = None
    B, S = 4, 64
    g = torch.Generator().manual_seed(100 + rank)
    base = torch.randint(0, 256, (S + 1,), generator=g)
    ids = base[:-1].repeat(B, 1).to(dev)
    labels = base[1:].repeat(B, 1).to(dev)
    ref_loss = float(full.forward_backward(ids, labels))
    experts = attach_expert_parallel(model, symm, rank, world, B * S)
    tr = EPTrainer(model, experts, lr=3e-3, weight_decay=0.0)
    model.flat.zero_grad()
    ep_loss = float(model.forward_backward(ids, labels))
    res = {"ref_loss": ref_loss, "ep_loss": ep_loss, "local_experts": int(model.layers[0].gate_up.shape[0])}
    # gradient of a replicated tensor matches the full model's on this rank's batch (before any cross-rank averaging)
    ga, gb = model.layers[0].qkv.main_grad, full.layers[0].qkv.main_grad
    res["g_qkv"] = float((ga - gb).abs().max() / gb.abs().max().clamp(min=1e-9))
    El = res["local_experts"]
    ge, gf = model.layers[0].down.main_grad, full.layers[0].down.main_grad[rank * El:(rank + 1) * El]
    res["g_down_has_remote_tokens"] = float((ge - gf).abs().max()) > 0      # the owner also sees the other rank's tokens
    model.flat.zero_grad()                      # the optimiser step leaves the gradients zeroed; start from that state
    losses = [tr.train_step(ids, labels) for _ in range(8)]
    res["losses"] = losses
    w = model.layers[0].qkv.data.float()
    ws = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(ws, w)
    res["replicated_in_sync"] = bool(all(torch.equal(ws[0], x) for x in ws))
    torch.cuda.synchronize()
    res["status"] = int(_lib.status_word(dev)[0].item())
    json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    dist.barrier()
    symm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
