"""Pipeline worker (gloo, CPU): 1F1B and GPipe over N stages must reproduce the single-process loss and gradients."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import TransformerConfig  # noqa: E402
from transformers_fusion_b200.models.dense import DenseModel  # noqa: E402
from transformers_fusion_b200.parallel.collectives import DistributedContext  # noqa: E402
from transformers_fusion_b200.parallel.pp import PipelineParallel  # noqa: E402


def tied_case(ctx, ids, labels):
    """Tied embedding / LM head: both end stages must hold the summed gradient, clip on the global norm and end one
    optimizer step with the same table as a single-process run."""
    from transformers_fusion_b200.engines.dense import OptimSuite
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=4, num_heads=4, ffn_hidden_size=64, max_seq_len=16,
                            tie_embeddings=True)
    ref = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=2)
    ref.flatten()
    ref.forward_backward(ids, labels)
    ro = OptimSuite("adamw", 1e-2, 0.0)
    ro.add_group(list(ref.parameters()), 1.0, 1.0)
    ref_norm = ro.clip(0.05)
    ref_emb_grad = ref.tok_embeddings.main_grad.clone()
    ro.step()
    m = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=2)
    pp = PipelineParallel(m, ctx.world_size, ctx.rank, ctx, num_microbatches=4)
    pp.run_1f1b(ids, labels)
    opt = OptimSuite("adamw", 1e-2, 0.0)
    opt.add_group(pp.owned_parameters(), 1.0, 1.0)
    norm = pp.clip_gradients(0.05)
    out = {"tied_norm_err": abs(norm - ref_norm) / ref_norm}
    if pp.first or pp.last:
        out["tied_grad_err"] = float((m.tok_embeddings.main_grad - ref_emb_grad).abs().max())
        opt.step()
        out["tied_param_err"] = float((m.tok_embeddings.data - ref.tok_embeddings.data).abs().max())
    return out


def main():
    out_dir = sys.argv[1]
    ctx = DistributedContext.init("gloo")
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=4, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 64, (8, 16), generator=g)
    labels = torch.roll(ids, -1, 1)
    labels[0, :3] = -100
    res = {}
    ref = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=1)
    ref.flatten()
    ref_loss = float(ref.forward_backward(ids, labels))
    for sched in ("gpipe", "1f1b", "1f1b_tied"):
        if sched == "1f1b_tied":
            res.update(tied_case(ctx, ids, labels))
            continue
        m = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=1)
        pp = PipelineParallel(m, ctx.world_size, ctx.rank, ctx, num_microbatches=4)
        pp.set_profiling(True)
        loss = pp.run_gpipe(ids, labels) if sched == "gpipe" else pp.run_1f1b(ids, labels)
        if pp.last:
            res[f"{sched}_loss_err"] = abs(float(loss) - ref_loss)
        err = 0.0
        name_of = {id(p): n for n, p in m.named_parameters()}
        refp = dict(ref.named_parameters())
        for p in pp.owned_parameters():
            n = name_of[id(p)]
            if n == "tok_embeddings" and cfg.tie_embeddings:
                continue
            err = max(err, float((p.main_grad - refp[n].main_grad).abs().max()))
        res[f"{sched}_grad_err"] = err
        res[f"{sched}_live"] = pp.max_live_microbatches(sched)
        assert not pp._saved
    # inference pass through the stages: the last stage's logits equal the single-process model's
    m = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=1)
    pp = PipelineParallel(m, ctx.world_size, ctx.rank, ctx, num_microbatches=4)
    logits = pp.forward(ids)
    if pp.last:
        with torch.no_grad():
            want = ref.forward(ids)
        res["fwd_logits_err"] = float((logits - want).abs().max())
        res["fwd_loss_err"] = abs(float(pp.compute_loss(logits, labels)) - ref_loss)
    else:
        assert logits is None
    res["two_call_loss"] = pp.forward_1f1b(ids, labels) is pp.backward_1f1b() and pp.micro_batch_queue_size() == 0
    res["stage_params"] = pp.model_param_count()
    json.dump(res, open(os.path.join(out_dir, f"rank{ctx.rank}.json"), "w"))
    ctx.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
