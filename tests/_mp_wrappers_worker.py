"""The reference's first-generation wrappers on two gloo ranks: tensor-parallel and pipeline forward equal the dense model;
parameter-server averaging; context accessors."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import TransformerConfig  # noqa: E402
from transformers_fusion_b200.models.dense import DenseModel  # noqa: E402
from transformers_fusion_b200.parallel.collectives import DistributedContext, ParameterServer, RingAllReduce  # noqa: E402
from transformers_fusion_b200.parallel.ddp import (DDPWrapper, DistributedDataParallel, PipelineParallelWrapper,  # noqa: E402
                                                   TensorParallelWrapper)


def main():
    out_dir = sys.argv[1]
    ctx = DistributedContext.init("gloo")
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(0))
    ref = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=1)
    with torch.no_grad():
        want = ref.forward(ids)
    res = {"is_main": ctx.is_main(), "mode0": ctx.mode}
    tpw = TensorParallelWrapper(DenseModel(cfg, device="cpu", dtype=torch.float32, seed=1), DistributedContext(ctx.rank, ctx.world_size))
    res["tp_err"] = float((tpw.forward(ids) - want).abs().max())
    res["tp_mode"] = tpw.context().mode
    res["split"] = list(tpw.split_linear(torch.arange(8.0).view(4, 2), 0).reshape(-1).tolist())
    ppw = PipelineParallelWrapper(DenseModel(cfg, device="cpu", dtype=torch.float32, seed=1), DistributedContext(ctx.rank, ctx.world_size))
    lg = ppw.forward(ids)
    res["pp_err"] = float((lg - want).abs().max()) if lg is not None else None
    ps = ParameterServer(num_shards=2).configure_world(ctx.world_size, ctx.rank, 1)
    ps.push("w", torch.full((4,), float(ctx.rank)))
    ps.average_parameters(1.0, ctx)
    res["ps_avg"] = ps.get_param("w").tolist()
    res["ps_node"] = [ps.is_ps_node(), ps.ps_node_id(), ps.num_ps_nodes()]
    ps.barrier(ctx)
    ring = RingAllReduce(ctx)
    res["ring"] = [ring.rank(), ring.world_size()]
    ring.barrier()
    ddp = DistributedDataParallel(DenseModel(cfg, device="cpu", dtype=torch.float32, seed=1), ctx)
    ddp.set_grad_accumulation_steps(2)
    ddp.forward_backward(ids, torch.roll(ids, -1, 1))
    res["ddp"] = [ddp.grad_accum_count(), ddp.grad_accumulation_steps(), ddp.rank(), ddp.world_size(), ddp.context() is ctx]
    ddp.reset_grad_accum_count()
    res["ddp_reset"] = ddp.grad_accum_count()
    res["wrapper_ctx"] = DDPWrapper(ref, ctx).context() is ctx
    json.dump(res, open(os.path.join(out_dir, f"rank{ctx.rank}.json"), "w"))
    ctx.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
