"""Worker for the sharded (ZeRO-3 x tensor-parallel) engine: dp x tp ranks must reproduce the losses and the weights of
a single-process run on the whole batch.  Runs on CPU with gloo (library collectives) or on GPUs (``fused`` / ``nccl``)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import TransformerConfig  # noqa: E402
from transformers_fusion_b200.models.dense import DenseModel  # noqa: E402
from transformers_fusion_b200.parallel.launch import init_parallel  # noqa: E402
from transformers_fusion_b200.parallel.sharded import Mesh, ShardedEngine  # noqa: E402
from transformers_fusion_b200.trainer.engine import TrainEngine  # noqa: E402


def main():
    out_dir, tp, comm = sys.argv[1], int(sys.argv[2]), sys.argv[3]
    tied = len(sys.argv) > 4 and sys.argv[4] == "tied"
    st = init_parallel(tp=tp, device="cpu" if comm == "gloo" else "auto")
    cuda = st.device.type == "cuda"
    dt = torch.bfloat16 if cuda else torch.float32
    if cuda:
        cfg = TransformerConfig(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=512,
                                max_seq_len=128, tie_embeddings=tied)
        B, S = 4 * st.dp, 128
    else:
        cfg = TransformerConfig(vocab_size=96, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=64,
                                max_seq_len=16, tie_embeddings=tied)
        B, S = 2 * st.dp, 16
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=g).to(st.device)
    labels = torch.roll(ids, -1, 1)
    # bf16 on GPUs: Adam turns rounding noise in near-zero gradients into full-size steps, so the weight comparison there
    # uses a small learning rate (the losses and the gradient norm carry the check)
    kw = dict(lr=1e-3 if cuda else 1e-2, betas=(0.9, 0.95), weight_decay=0.0, max_grad_norm=0.5)
    ref = DenseModel(cfg, device=st.device, dtype=dt, seed=3)
    src = DenseModel(cfg, device=st.device, dtype=dt, seed=3)
    dp_heap = tp_heap = None
    if comm in ("fused", "fused_in_gemm"):
        from transformers_fusion_b200.parallel.symm import SymmetricHeap
        if st.dp > 1:
            dp_heap = SymmetricHeap(st.dp_rank, st.dp, st.device, group=st.dp_group)
        if st.tp > 1:
            tp_heap = SymmetricHeap(st.tp_rank, st.tp, st.device, group=st.tp_group)
    mesh = Mesh(st.dp_rank, st.dp, st.tp_rank, st.tp, st.dp_group, st.tp_group, None)
    gather = "fused" if comm == "fused_in_gemm" else "prefetch"
    eng = ShardedEngine.from_dense(src, mesh, comm={"gloo": "nccl", "fused_in_gemm": "fused"}.get(comm, comm), dp_heap=dp_heap,
                                   tp_heap=tp_heap, loss_chunk_tokens=256, gather=gather, **kw)
    ref_eng = TrainEngine(ref, zero_stage=0, comm="none", **kw)
    ref_eng.world, ref_eng.zero_stage = 1, 0
    per = B // st.dp
    my_ids, my_lab = ids[st.dp_rank * per:(st.dp_rank + 1) * per], labels[st.dp_rank * per:(st.dp_rank + 1) * per]
    res = {"loss_err": [], "gathers": 0}
    for step in range(3):
        # single-process statement of the same step: the whole batch on one model (ranks run it redundantly)
        ref.flat.grads.zero_()
        ref_loss = ref.forward_backward(ids, labels)
        ref_eng.opt.stage_hyper(None)
        ref_eng.opt.step(staged=True)
        loss = eng.train_step(my_ids, my_lab).detach().float().reshape(1).clone()
        if st.dp > 1:
            dist.all_reduce(loss, group=st.dp_group)
            loss /= st.dp
        res["loss_err"].append(abs(float(loss) - float(ref_loss)))
    if cuda:
        torch.cuda.synchronize()
        from transformers_fusion_b200.ops import _lib
        _lib.check_status(st.device)
    res["gathers"] = eng.gathers
    eng.export_to(src)
    werr = 0.0
    refp = dict(ref.named_parameters())
    for n, p in src.named_parameters():
        scale = float(refp[n].float().abs().max()) + 1e-6
        werr = max(werr, float((p.float() - refp[n].float()).abs().max()) / scale)
    res["weight_err"] = werr
    res["losses"] = [float(x) for x in res.get("losses", [])]
    res["grad_norm"] = float(eng.last_grad_norm)
    res["ref_grad_norm"] = float(ref_eng.opt.grad_norm)
    mp = eng.memory_profile()
    res["mem_total"], res["mem_unsharded"] = mp["total"], mp["unsharded_total"]
    json.dump(res, open(os.path.join(out_dir, f"rank{st.rank}.json"), "w"))
    dist.barrier()
    if cuda:
        for h in (dp_heap, tp_heap):
            if h is not None:
                h.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
