"""Host-side logic of the expert-parallel trainer: which slices of the flat gradient buffer are all-reduced."""
import torch

from transformers_fusion_b200.models.config import MoEConfig
from transformers_fusion_b200.models.moe import MoEModel
from transformers_fusion_b200.parallel.ep_model import EPTrainer


def _trainer(model):
    experts = [p for blk in model.layers if hasattr(blk, "router") for p in (blk.gate_up, blk.down)]
    ids = {id(p) for p in experts}
    t = EPTrainer.__new__(EPTrainer)          # no optimiser / process group needed for the run computation
    t.model, t.experts, t._runs = model, experts, None
    t.shared = [p for p in model.parameters() if id(p) not in ids]
    return t


def test_shared_runs_cover_replicated_tensors_and_skip_experts():
    cfg = MoEConfig(vocab_size=512, hidden_size=64, num_layers=3, num_heads=4, ffn_hidden_size=128, max_seq_len=64,
                    num_experts=4, top_k=2, expert_hidden_size=64, tie_embeddings=True)
    m = MoEModel(cfg, device="cpu", dtype=torch.bfloat16, seed=0)
    if m.flat is None:
        m.flatten()
    t = _trainer(m)
    runs = t._shared_runs()
    assert 1 <= len(runs) < len(t.shared)                       # merged: far fewer collectives than tensors
    flat = m.flat.grads
    mark = torch.zeros_like(flat)
    for r in runs:
        assert r.data_ptr() >= flat.data_ptr() and r.is_contiguous()
        r.add_(1.0)                                             # what an all-reduce would touch
    mark.copy_(flat)
    for p in t.shared:
        assert bool((p.main_grad == 1).all())                   # every replicated gradient is covered exactly once
    for p in t.experts:
        assert bool((p.main_grad == 0).all())                   # no expert gradient is touched
    assert float(mark.max()) == 1.0
    flat.zero_()
    assert t._shared_runs() is runs                             # computed once
