"""Engine facades for fine-tuning, QAT, mixed precision and continual learning."""
import math

import pytest
import torch

from transformers_fusion_b200.engines import dense_extras as X
from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.trainer.continual import ContinualEngineConfig, ECCState
from transformers_fusion_b200.trainer.finetune import FineTuner
from transformers_fusion_b200.trainer.trainer import DataLoader, TrainConfig, Trainer


def tiny(seed=0):
    return DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=48, max_seq_len=32, init_std=0.1),
                      dtype=torch.float32, seed=seed)


def loader(seed=0):
    base = torch.randint(0, 64, (16,), generator=torch.Generator().manual_seed(seed))
    return DataLoader(tokens=base.repeat(60), batch_size=4, seq_length=16)


def test_lora_engine_and_finetune_runner():
    eng = X.LoRAEngine(X.LoRAConfig(rank=4, alpha=8.0))
    eng.attach("down", 16, 8)
    x = torch.randn(5, 16)
    assert float(eng.forward("down", x).detach().abs().sum()) == 0.0 and eng.trainable_params() == 4 * 16 + 8 * 4 and eng.config().rank == 4
    with torch.no_grad():
        eng.layers["down"].B.normal_()
    w = torch.randn(8, 16)
    merged = eng.merge_into(w.clone(), "down")
    assert torch.allclose(x @ merged.t(), x @ w.t() + eng.forward("down", x), atol=1e-5)
    half = eng.merge_into(w.clone(), "down", 0.5)
    assert torch.allclose(half - w, (merged - w) * 0.5, atol=1e-6)
    eng.zero("down")
    assert float(eng.forward("down", x).detach().abs().sum()) == 0.0
    with pytest.raises(KeyError):
        eng.forward("nope", x)
    m = tiny()
    r = X.FinetuneRunner(FineTuner(m, lr=1e-3, fmt=None))
    dl = loader()
    st = r.fine_tune(dl, max_batches=5)
    assert st.steps == 5 and st.tokens == 5 * 64 and st.tok_per_sec > 0 and math.isfinite(st.last_loss)
    g = torch.zeros(1024)
    g[300] = 1.0
    assert r.trainable_blocks(g, 1e-6, 256) == [1] and r.stats().trainable_blocks == 1


def test_qat_engine_schedule_and_mixed_precision():
    m = tiny()
    t = Trainer(m).compile("adamw", TrainConfig(batch_size=4, seq_length=16, learning_rate=1e-3, warmup_steps=0, zero_stage=0))
    q = X.QATEngine(bits=4).attach(t)
    q.set_schedule(2, 4)
    dl = loader()
    on = []
    for _ in range(5):
        on.append(q.sync())
        t.train_step(*dl.next_batch())
    assert on == [False, False, True, True, False] and q.stats().steps == 2 and not t.qat_enabled() and q.active_at(3) and not q.active_at(4)
    w = torch.randn(64, 64)
    fq4 = q.fake_quantize(w)
    q8 = X.QATEngine(bits=8)
    assert torch.unique(fq4).numel() <= 15 and q8.sqnr_db(w, q8.fake_quantize(w)) > q.sqnr_db(w, fq4) + 15      # about 6 dB per bit
    st = q8.calibrate([w, 2 * w])
    assert st.mean_sqnr_db > 30 and st.mean_scale == pytest.approx(1.5 * float(w.abs().max()) / 127, rel=1e-5) and q8.step_scales() == st.mean_scale
    assert q.inner().bits_for_format() == 4
    p = torch.nn.Parameter(torch.zeros(4))
    mp = X.MixedPrecision(8.0, interval=2)
    p.grad = torch.full((4,), 16.0)
    assert mp.step([p]) and torch.equal(p.grad, torch.full((4,), 2.0)) and mp.scale() == 8.0
    p.grad = torch.tensor([1.0, float("inf"), 0.0, 0.0])
    assert not mp.step([p]) and mp.scale() == 4.0 and mp.stats().overflows == 1
    p.grad = torch.ones(4)
    mp.step([p]), mp.step([p])
    assert mp.scale() == 8.0 and mp.stats().steps == 4


def test_continual_runner_and_ewc_probe():
    ecc = ECCState()
    w = torch.ones(8)
    X.EWCProbe.anchor(ecc, w)
    X.EWCProbe.accumulate_fisher(ecc, torch.full((8,), 2.0), 1.0)
    assert X.EWCProbe.penalty(ecc, w, 1.0) == 0.0 and X.EWCProbe.penalty(ecc, w + 1.0, 1.0) > 0
    m = tiny()
    t = Trainer(m).compile("adamw", TrainConfig(batch_size=4, seq_length=16, learning_rate=2e-3, warmup_steps=0, zero_stage=0))
    r = X.ContinualRunner(t, ContinualEngineConfig(ecc_lambda=10.0, ecc_alpha=0.1, replay_capacity=64))
    r.set_replay_ratio(0.25), r.set_ewc_lambda(5.0)
    assert r.engine() is t.continual_engine() and r.engine().cfg.ecc_lambda == 5.0 and r.ewc_penalty() == 0.0
    a, b = loader(0), loader(1)
    for _ in range(6):
        r.train_step_mixed(*a.next_batch())
    a.reset()
    r.on_task_boundary(1, a)
    for _ in range(6):
        loss = r.train_step_mixed(*b.next_batch(), replay_ratio=0.5)
    s = r.stats()
    assert s.task_id == 1 and s.steps == 12 and math.isfinite(loss) and s.ewc_penalty > 0 and t.replay_ratio == 0.5
    ids, lab = b.next_batch()
    mixed, _ = r.replay_mix(ids, lab, 0.5)
    assert mixed.shape == ids.shape and not torch.equal(mixed, ids)
    assert r.eval_forgetting() >= 0.0 and 0.0 <= r.stats().stability <= 1.0
