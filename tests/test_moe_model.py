"""MoE model: training reduces the loss, metrics are populated, variants run, checkpoint names follow
the reference, pipeline writes per-epoch files (tiny shapes as in the reference's test_moe_training:
V64 H32 L1 E4 top-2, AdamW)."""
import json

import pytest
import torch

from transformers_fusion_b200.models.config import MoEConfig
from transformers_fusion_b200.models.moe import VARIANTS, MoEModel
from transformers_fusion_b200.quant import codec
from transformers_fusion_b200.trainer.moe_trainer import MoETrainConfig, MoETrainer, MoETrainingPipeline
from transformers_fusion_b200.trainer.trainer import DataLoader


def cfg(**kw):
    base = dict(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=48, max_seq_len=32,
                num_experts=4, top_k=2, init_std=0.1)
    base.update(kw)
    return MoEConfig(**base)


def stream():
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, 64, (16,), generator=g).repeat(300)


def test_moe_training_reduces_loss_and_reports_metrics():
    m = MoEModel(cfg(), dtype=torch.float32, seed=1)
    t = MoETrainer(m).compile("adamw", MoETrainConfig(batch_size=4, seq_length=16, learning_rate=1e-2, warmup_steps=0,
                                                     lr_schedule="CONSTANT"))
    dl = DataLoader(tokens=stream(), batch_size=4, seq_length=16)
    losses = [t.train_step(*dl.next_batch()) for _ in range(40)]
    assert losses[-1] < losses[0] - 0.3 and all(x == x for x in losses)
    mt = t.metrics()
    assert len(mt.expert_utilization) == 4 and abs(sum(mt.expert_utilization) - 1.0) < 1e-4
    assert mt.aux_loss > 0 and mt.load_imbalance >= 1.0
    # the router receives gradient through the auxiliary losses and the combine weights
    m.flat.zero_grad()
    m.forward_backward(*dl.next_batch())
    assert m.layers[0].router.main_grad.abs().sum() > 0


@pytest.mark.parametrize("variant", ["SPARSE_TOP1", "SOFT_MIXTURE", "HASH_ROUTED", "DEEPSEEK_MOE", "SHARED_EXPERT",
                                     "RESIDUAL_MOE", "GATING_DROPOUT"])
def test_variants_run(variant):
    assert variant in VARIANTS
    c = cfg(variant=variant, num_shared_experts=1 if variant == "SHARED_EXPERT" else 0)
    m = MoEModel(c, dtype=torch.float32, seed=2)
    m.flatten()
    ids = torch.randint(0, 64, (2, 16))
    loss = m.forward_backward(ids, torch.roll(ids, -1, 1))
    assert torch.isfinite(loss) and torch.isfinite(m.flat.grads).all() and m.flat.grads.abs().sum() > 0


def test_checkpoint_names_and_pipeline(tmp_path):
    m = MoEModel(cfg(num_shared_experts=1), dtype=torch.float32, seed=3)
    p = tmp_path / "moe.quant"
    codec.save_model(m, p)
    names = codec.QuantReader(p).tensor_names()
    assert "layers.0.moe.router.weight" in names and "layers.0.moe.expert.3.down_proj.weight" in names
    assert "layers.0.shared_expert.gate_proj.weight" in names
    t = MoETrainer(m).compile("adamw", MoETrainConfig(batch_size=2, seq_length=16, learning_rate=1e-3))
    hist = MoETrainingPipeline(t, str(tmp_path / "run")).run(DataLoader(tokens=stream(), batch_size=2, seq_length=16), 2, 3)
    assert len(hist) == 2 and (tmp_path / "run" / "moe_epoch1.quant").exists()
    assert json.load(open(tmp_path / "run" / "moe_epoch0.json"))["num_experts"] == 4
