"""Worker for the tensor-parallel model tests: the TP + SP model against the single-rank DenseModel on the same batch
(loss, sharded and replicated gradients), a few optimiser steps, and the shard gather.  argv: <out_dir> <cpu|cuda>."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from transformers_fusion_b200.models.config import TransformerConfig  # noqa: E402
from transformers_fusion_b200.models.dense import DenseModel  # noqa: E402
from transformers_fusion_b200.parallel.tp_model import TPDenseModel, TPGroup, TPTrainer  # noqa: E402


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(1e-9, b.float().abs().max().item())


def main():
    out_dir, where = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    ctx = symm = None
    if where == "cuda":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=dev)
        dtype, B, S, H, heads, Fh = torch.bfloat16, 2, 128 * world, 256, 4, 512
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        dtype, B, S, H, heads, Fh = torch.float32, 2, 8 * world, 32, 4, 48 * world
    cfg = TransformerConfig(vocab_size=128, hidden_size=H, num_layers=2, num_heads=heads, num_kv_heads=2 * (world // 2) or 2,
                            ffn_hidden_size=Fh, max_seq_len=S, init_std=0.08)
    if cfg.num_kv_heads % world:
        cfg.num_kv_heads = heads
    dense = DenseModel(cfg, device=dev, dtype=dtype, seed=3)
    if where == "cuda":
        from transformers_fusion_b200.parallel.symm import SymmetricHeap
        from transformers_fusion_b200.parallel.tp import TpContext
        symm = SymmetricHeap(rank, world, dev)
        T = B * S
        widest = max(H, 2 * Fh // world, (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim // world)
        ctx = TpContext(symm, rank, world, T, max(H, widest), max(H, widest), copy_ctas=8)
    tp = TPGroup(rank, world, None, ctx)
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, 128, (B, S + 1), generator=g)
    ids, labels = ids[:, :-1].contiguous().to(dev), ids[:, 1:].contiguous().to(dev)
    res = {}
    # reference: the whole model on this rank
    dense.flatten()
    ref_loss = float(dense.forward_backward(ids, labels))
    tpm = TPDenseModel(dense, tp)
    loss = float(tpm.forward_backward(ids, labels))
    res["loss_err"] = abs(loss - ref_loss) / abs(ref_loss)
    D, W = cfg.head_dim, world
    l0, d0 = tpm.layers[0], dense.layers[0]
    nq, nkv = cfg.num_heads * D, cfg.num_kv_heads * D
    hq, hkv = l0.hq * D, l0.hkv * D
    gq = d0.qkv.main_grad
    want_qkv = torch.cat([gq[:nq][rank * hq:(rank + 1) * hq], gq[nq:nq + nkv][rank * hkv:(rank + 1) * hkv],
                          gq[nq + nkv:][rank * hkv:(rank + 1) * hkv]], 0)
    res["g_qkv"] = rel(l0.qkv.main_grad, want_qkv)
    res["g_o"] = rel(l0.o.main_grad, d0.o.main_grad[:, rank * hq:(rank + 1) * hq])
    Fl = cfg.ffn_hidden_size // W
    res["g_down"] = rel(l0.down.main_grad, d0.down.main_grad[:, rank * Fl:(rank + 1) * Fl])
    ggu = d0.gate_up.main_grad
    Fh_ = cfg.ffn_hidden_size
    res["g_gate_up"] = rel(l0.gate_up.main_grad, torch.cat([ggu[:Fh_][rank * Fl:(rank + 1) * Fl], ggu[Fh_:][rank * Fl:(rank + 1) * Fl]], 0))
    res["g_attn_norm"] = rel(l0.attention_norm.main_grad, d0.attention_norm.main_grad)
    res["g_final_norm"] = rel(tpm.norm.main_grad, dense.norm.main_grad)
    res["g_embed"] = rel(tpm.tok_embeddings.main_grad, dense.tok_embeddings.main_grad + (0 if not tpm.tied else 0))
    # a few optimiser steps: the loss goes down and every rank sees the same value
    for p in tpm.parameters():
        p.main_grad.zero_()
    tr = TPTrainer(tpm, lr=3e-3 if where == "cpu" else 1e-3, weight_decay=0.0)
    losses = [tr.train_step(ids, labels) for _ in range(6)]
    res["losses"] = losses
    full = tpm.gather_into()
    with torch.no_grad():
        logits = full(ids).float()
        res["gathered_loss"] = float(torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1)))
    if where == "cuda":
        from transformers_fusion_b200.ops import _lib
        torch.cuda.synchronize()
        res["status"] = int(_lib.status_word(dev)[0].item())
    json.dump(res, open(os.path.join(out_dir, f"rank{rank}.json"), "w"))
    dist.barrier()
    if symm is not None:
        symm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
