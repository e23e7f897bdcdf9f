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


def test_moe_trainer_accumulates_fresh_micro_batches_and_scales_loss():
    """Two micro-batches drawn from the loader under a loss scale give the same update as one step on both batches."""
    def make():
        m = MoEModel(cfg(), dtype=torch.float32, seed=5)
        return m
    dl_a = DataLoader(tokens=stream(), batch_size=2, seq_length=16)
    dl_b = DataLoader(tokens=stream(), batch_size=2, seq_length=16)
    kw = dict(batch_size=2, seq_length=16, learning_rate=1e-2, warmup_steps=0, lr_schedule="CONSTANT", max_grad_norm=0.0)
    ta = MoETrainer(make()).compile("sgd", MoETrainConfig(grad_accum_steps=2, mixed_precision=True, loss_scale=64.0, **kw))
    assert ta.mixed_precision_active() and ta.gradient_accumulation_steps() == 2
    first = dl_a.next_batch()
    ta.train_step(*first, loader=dl_a)
    assert ta.metrics().tokens_processed == 2 * 2 * 16
    assert ta.loss_scale == pytest.approx(64.0 * 1.01)                  # a clean step grows the scale by 1 %
    tb = MoETrainer(make()).compile("sgd", MoETrainConfig(**kw))
    b0, b1 = dl_b.next_batch(), dl_b.next_batch()
    tb.train_step(torch.cat([b0[0], b1[0]]), torch.cat([b0[1], b1[1]]))
    # the auxiliary terms are per micro-batch statistics, so the two routes agree up to their small weight
    assert torch.allclose(ta.model.flat.params, tb.model.flat.params, atol=2e-3)
    mt = ta.metrics()
    assert mt.load_balance_loss >= 1.0 - 1e-3 and mt.z_loss > 0 and mt.total_loss == pytest.approx(mt.loss + mt.aux_loss)
    assert mt.num_experts_used >= 2 and 0 < mt.mean_expert_utilization <= 1 and mt.active_params < mt.total_params
    # an overflowing step is dropped and halves the scale
    scale = ta.loss_scale
    ta.model.layers[0].down.data[0, 0, 0] = float("nan")
    ta._mp_master.copy_(ta.model.flat.params.float())              # the forward pass reads the master values
    before = ta.model.flat.params.clone()
    ta.train_step(*dl_a.next_batch(), loader=dl_a)
    assert ta.loss_scale == pytest.approx(scale / 2)
    same = torch.isnan(before) | (ta.model.flat.params == before)
    assert bool(same.all())


def test_moe_trainer_master_copy_ema_and_aux_term():
    m = MoEModel(cfg(), dtype=torch.bfloat16, seed=6)
    t = MoETrainer(m).compile("sgd", MoETrainConfig(batch_size=2, seq_length=16, learning_rate=1e-4, warmup_steps=0,
                                                   lr_schedule="CONSTANT", mixed_precision=True, loss_scale=1.0))
    dl = DataLoader(tokens=stream(), batch_size=2, seq_length=16)
    start = t._mp_master.clone()
    for _ in range(3):
        t.train_step(*dl.next_batch())
    assert (t._mp_master - start).abs().max() > 0
    assert torch.equal(m.flat.params, m.flat.params) and (t._mp_master.to(torch.bfloat16).float() - m.flat.params.float()).abs().max() < 1e-2
    t.ema_init(0.5)
    t.train_step(*dl.next_batch())
    t.ema_step()
    avg = t.ema.shadow.clone()
    t.ema_apply()
    assert torch.equal(m.flat.params.float(), avg.to(torch.bfloat16).float())
    # the canonical balance term: uniform routing with uniform probabilities gives exactly 1
    E = 4
    logits = torch.zeros(8, E)
    idx = torch.arange(8).remainder(E).reshape(8, 1)
    assert t.compute_aux_loss(logits, idx) == pytest.approx(1.0)
    assert t.compute_aux_loss(logits, torch.zeros(8, dtype=torch.long)) == pytest.approx(1.0)   # P uniform: f does not matter
    skew = torch.zeros(8, E)
    skew[:, 0] = 4.0
    assert t.compute_aux_loss(skew, torch.zeros(8, 1, dtype=torch.long)) > 3.0                    # everything on one expert


def test_moe_pipeline_from_files_early_stop_and_report(tmp_path):
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    text = ("the quick brown fox jumps over the lazy dog. " * 40)
    (tmp_path / "train.txt").write_text(text)
    (tmp_path / "val.txt").write_text(text[:600])
    m = MoEModel(cfg(vocab_size=260), dtype=torch.float32, seed=7)
    tr = MoETrainer(m, ByteTokenizer())
    pipe = MoETrainingPipeline(tr, str(tmp_path / "ck"), train_path=str(tmp_path / "train.txt"), val_path=str(tmp_path / "val.txt"))
    pipe.set_log_file(str(tmp_path / "log.txt"))
    pipe.configure(MoETrainConfig(batch_size=2, seq_length=16, learning_rate=0.0, warmup_steps=0, max_steps=2, epochs=6,
                                  log_interval=1))
    pipe.patience, pipe.min_delta = 2, 1e-3
    hist = pipe.run(6)
    # a learning rate of (almost) zero cannot improve the validation loss: epoch 0 sets the best, epochs 1 and 2 exhaust the patience
    assert len(hist) == 3 and hist[-1]["val_loss"] is not None
    assert (tmp_path / "ck" / "moe_epoch2.quant").exists() and json.load(open(tmp_path / "ck" / "moe_epoch2.json"))["top_k"] == 2
    log = (tmp_path / "log.txt").read_text()
    assert "Step 1 |" in log and "Early stop" in log
    rep = pipe.status_report()
    assert "MoE Training Report" in rep and "Experts: 4 (top-2)" in rep


def test_stand_alone_mixture_layers_under_the_reference_class_names():
    from transformers_fusion_b200.models import moe as M
    cfg = M.MoEAllConfig(num_experts=8, top_k=2, expert_hidden=32)
    x = torch.randn(2, 6, 16)
    assert len(M.MOE_LAYER_CLASSES) == 25 and set(M.MOE_LAYER_CLASSES) <= set(M.VARIANTS)
    for variant, cls in M.MOE_LAYER_CLASSES.items():
        layer = cls(16, cfg)
        xin = x.clone().requires_grad_(True)
        out = layer(xin)
        (out.output.float().sum() + out.aux_loss).backward()
        assert out.output.shape == x.shape and torch.isfinite(out.output).all() and xin.grad is not None, variant
        assert all(not n.startswith("block.qkv") for n, _ in layer.named_parameters())       # no attention half
    sp = M.SparseMoE(16, cfg)
    o = sp(x, training=False)
    assert o.expert_indices.shape == (12, 2) and o.router_logits.shape == (12, 8) and sp.router_weight.shape == (8, 16) and len(sp.experts) == 8
    # the layer is the weighted sum of its chosen experts
    logits = (x.reshape(-1, 16) @ sp.router_weight.t()).detach()
    w, idx = torch.softmax(logits.float(), -1).topk(2, -1)
    w = w / w.sum(-1, keepdim=True) if sp.block.cfg.renormalize_topk else w
    want = torch.zeros(12, 16)
    for t in range(12):
        for j in range(2):
            gu, dn = sp.experts[int(idx[t, j])]
            h = x.reshape(-1, 16)[t] @ gu.t()
            want[t] += w[t, j] * ((torch.nn.functional.silu(h[:32]) * h[32:]) @ dn.t())
    assert torch.allclose(o.output.reshape(12, 16), want, atol=1e-4)
    gates = torch.softmax(logits, -1)
    assert float(sp.load_balance_loss(gates, idx)) > 0 and float(sp.z_loss(logits)) > 0 and sp.compute_capacity(64) >= 64 * 2 // 8
    blob = sp.export_weights()
    other = M.SparseMoE(16, cfg, seed=5)
    assert not torch.allclose(other(x).output, o.output)
    other.import_weights(blob)
    assert torch.allclose(other(x, training=False).output, o.output)
    with pytest.raises(ValueError):
        other.import_weights(blob[:-4])
    res = M.ResidualMoE(16, cfg)
    plain = M.SparseMoE(16, cfg)
    assert torch.allclose(res(x, False).output, plain(x, False).output + x, atol=1e-5)       # same seed: same experts, plus the input
