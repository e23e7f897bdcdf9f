"""Worker of test_ep_replicas: two CPU ranks, every rank holds all experts (expert-parallel degree 1, two replicas), so the
trainer's replica reduction must reproduce plain data parallelism over the combined batch."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import TransformerConfig  # noqa: E402
from transformers_fusion_b200.models.moe import MoEAllConfig, create_moe_variant  # noqa: E402
from transformers_fusion_b200.parallel.ep_model import EPTrainer  # noqa: E402


def make():
    base = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    m = create_moe_variant("SPARSE_TOPK", base, MoEAllConfig(num_experts=4, top_k=2, expert_hidden=32, load_balance_weight=0.0),
                           device="cpu", dtype=torch.float32, seed=0)
    m.flatten()
    return m


def main():
    out_dir = sys.argv[1]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = 0
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("gloo")
        rank = dist.get_rank()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 64, (4, 16), generator=g)
    lab = torch.roll(ids, -1, 1)
    m = make()
    experts = [p for blk in m.layers for p in (blk.gate_up, blk.down)]
    tr = EPTrainer(m, experts, lr=1e-2, weight_decay=0.0, max_grad_norm=1.0,
                   replica_group=dist.group.WORLD if world > 1 else None, replicas=world)
    per = ids.shape[0] // world
    losses = [tr.train_step(ids[rank * per:(rank + 1) * per], lab[rank * per:(rank + 1) * per]) for _ in range(3)]
    tag = f"w{world}_rank{rank}"
    json.dump({"losses": losses, "norm": tr.grad_norm}, open(os.path.join(out_dir, tag + ".json"), "w"))
    torch.save([p.detach().clone() for p in m.parameters()], os.path.join(out_dir, tag + ".pt"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
