"""Replicated-token expert parallelism on CPU ranks (gloo): logits, loss and gradients equal the single-process model."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import MoEConfig  # noqa: E402
from transformers_fusion_b200.models.moe import MoEModel  # noqa: E402
from transformers_fusion_b200.parallel.collectives import DistributedContext  # noqa: E402
from transformers_fusion_b200.parallel.ep_model import ModelExpertParallel  # noqa: E402


def main():
    out_dir = sys.argv[1]
    ctx = DistributedContext.init("gloo")
    cfg = MoEConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, ffn_hidden_size=48, max_seq_len=32,
                    num_experts=4, top_k=2, init_std=0.1)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 64, (2, 16), generator=g)
    labels = torch.roll(ids, -1, 1)
    ref = MoEModel(cfg, dtype=torch.float32, seed=1)
    ref.flatten()
    with torch.no_grad():
        want = ref.forward(ids)
    ref_loss = float(ref.forward_backward(ids, labels))
    m = MoEModel(cfg, dtype=torch.float32, seed=1)
    m.flatten()
    ep = ModelExpertParallel(4, ctx.world_size, ctx.rank, ctx)
    with torch.no_grad():
        got = ep.forward_with_parallel(m, ids)
    loss = float(ep.forward_backward(m, ids, labels))
    # before the sync an expert's gradient exists on its owner only
    own = ep.local_experts()
    other = [e for e in range(4) if e not in own]
    res = {"logits_err": float((got - want).abs().max()), "loss_err": abs(loss - ref_loss),
           "foreign_grad": float(m.layers[0].gate_up.main_grad[other].abs().max()) if other else 0.0,
           "local": own, "n_local": ep.num_local_experts()}
    ep.sync_gradients(m)
    err = 0.0
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        err = max(err, float((p.main_grad - q.main_grad).abs().max()))
    res["grad_err"] = err
    x = torch.full((2, 3), float(ctx.rank))
    res["gathered"] = ep.alltoall_experts(x)[:, 0].tolist()
    json.dump(res, open(os.path.join(out_dir, f"rank{ctx.rank}.json"), "w"))
    ctx.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
