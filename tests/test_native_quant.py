import math

import pytest
import torch

from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.trainer import training_utils as U
from transformers_fusion_b200.trainer.native_quant import Q1, Q4, Q8, NativeQUANTTrainer, NativeQWeightStore, NativeTrainConfig


def test_store_allocation_and_roundtrip():
    torch.manual_seed(0)
    w = torch.randn(128 * 100 + 17) * 0.1
    sens = torch.zeros_like(w)
    sens[: 128 * 2] = 5.0                                  # two very sensitive blocks
    st = NativeQWeightStore(w.numel(), 128)
    st.initialize(w, sens, 0.02, 0.9)
    c = st.counts()
    assert c[Q8] == 2 and c[Q1] == 91 and c[Q4] == 8 and int(st.formats[0]) == Q8 and int(st.formats[1]) == Q8
    d = st.dequantize()
    assert d.shape == w.shape
    e8 = (d[:256] - w[:256]).abs().max() / w[:256].abs().max()
    assert e8 < 0.03                                       # 8-bit blocks are close
    assert set(torch.unique(st.indices.view(-1, 128)[5]).tolist()) <= {0, 1, 2}
    assert 2.0 < st.bits_per_weight() < 3.0
    assert st.get_weight(3) == pytest.approx(float(d[3]))
    assert st.block_size() == 128 and st.get_format(0) == Q8 and st.get_format(5 * 128 + 3) == int(st.formats[5])
    i = 5 * 128 + 3
    assert st.get_index(i) == int(st.indices[i]) and st.get_scale(i) == float(st.scales[5])
    assert st.indices_data() is st.indices and st.block_scales_data() is st.scales and st.formats_data() is st.formats
    assert NativeQWeightStore.global_codebook().numel() == 256 and NativeQWeightStore.global_quant4_codebook().numel() == 16
    assert torch.equal(NativeQWeightStore.global_codebook(), st.cb8)


def test_quant_update_moves_toward_target():
    torch.manual_seed(1)
    tgt = torch.randn(128 * 8) * 0.1
    st = NativeQWeightStore(tgt.numel(), 128)
    st.initialize(tgt + torch.randn_like(tgt) * 0.1, None, 0.0, 0.0)  # all 4-bit, starting from a noisy copy
    e0 = float(((st.dequantize() - tgt) ** 2).mean())
    frozen = []
    for _ in range(300):
        g = 2 * (st.dequantize() - tgt)                    # gradient of the squared error
        frozen.append(st.apply_quant_update(g, 1e-2, 2e-2))
    e1 = float(((st.dequantize() - tgt) ** 2).mean())
    assert e1 < 0.05 * e0 and 0.2 < frozen[-1] <= 1.0       # converged onto the 4-bit grid; the rest oscillates between neighbours


def test_native_trainer_runs_through_transition(tmp_path):
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    m = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0)
    tr = NativeQUANTTrainer(m, NativeTrainConfig(warmup_steps=10, frac_quant8=0.1, frac_quant=0.5, lr_scale=1e-3, lr_weight=2e-2,
                                                 warmup_lr=5e-2, weight_decay=0.0))
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 64, (4, 16), generator=g)
    labels = torch.roll(ids, -1, 1)
    ms = [tr.train_step(ids, labels) for _ in range(40)]
    assert not math.isnan(ms[-1].loss) and tr.native
    assert ms[9].loss < ms[0].loss                          # warm-up learns
    assert ms[-1].quant8_count > 0 and ms[-1].quant1_count > 0 and ms[-1].quant_count > 0
    assert min(x.loss for x in ms[12:]) <= ms[11].loss + 0.05 and 0 < ms[-1].frozen_fraction <= 1
    tr.save_checkpoint(str(tmp_path / "n.pt"))
    m2 = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=5)
    t2 = NativeQUANTTrainer(m2, tr.cfg)
    t2.load_checkpoint(str(tmp_path / "n.pt"))
    assert torch.equal(m2.flat.params, m.flat.params) and t2.native
    # the warm-up as one call: stops after warmup_steps batches and switches to the quantised store
    t3 = NativeQUANTTrainer(DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0), tr.config())
    assert t3.config() is tr.cfg and math.isfinite(t3.warmup_phase([(ids, labels)] * 25)) and t3.native and t3.step_count == 10
    t4 = NativeQUANTTrainer(DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0), tr.config())
    t4.warmup_phase([(ids, labels)] * 3)
    assert t4.native and t4.step_count == 3                    # fewer batches than warm-up steps: still ends in the store


def test_training_utils():
    s = U.MixedPrecisionScaler(128, interval=2)
    assert s.update(True) == 64 and s.update(False) == 64 and s.update(False) == 128
    assert U.MixedPrecisionScaler.has_overflow(torch.tensor([1.0, float("inf")]))
    p = torch.nn.Parameter(torch.ones(4))
    ema = U.EMAWeightAveraging([p], 0.5)
    p.data.fill_(3.0)
    ema.update()
    ema.apply()
    assert torch.allclose(p.data, torch.full((4,), 2.0))
    ema.restore()
    assert torch.allclose(p.data, torch.full((4,), 3.0))
    es = U.EarlyStopping(patience=2)
    assert [es.step(v) for v in (1.0, 0.9, 0.95, 0.96)] == [False, False, False, True]
    w = U.LearningRateWarmup(1.0, 10)
    assert w.lr(0) == pytest.approx(0.1) and w.lr(20) == 1.0
    we = U.LearningRateWarmup(1.0, 10, "exponential")
    assert 0 < we.lr(0) < we.lr(5) < we.lr(9) <= 1.0 + 1e-6
    acc = U.GradientAccumulator(3)
    assert [acc.accumulate() for _ in range(6)] == [False, False, True, False, False, True]
    mt = U.MetricTracker()
    for v in (3, 2, 1):
        mt.add("loss", v)
    assert mt.mean("loss") == 2 and mt.best("loss") == 1
    logits = torch.randn(2, 5, 11)
    labels = torch.randint(0, 11, (2, 5))
    labels[0, 0] = -100
    assert U.focal_loss(logits, labels, gamma=0.0) == pytest.approx(float(U.cross_entropy_loss(logits, labels)), rel=1e-5)
    assert float(U.rdrop_loss(logits, logits, labels)) == pytest.approx(float(U.cross_entropy_loss(logits, labels)), rel=1e-5)
    e = torch.randn(6, 8)
    assert float(U.infonce_loss(e, e, 0.05)) < float(U.infonce_loss(e, torch.randn(6, 8), 0.05))
    assert float(U.z_loss(logits)) > 0 and float(U.mse_loss(e, e)) == 0
    heads = [torch.randn(11, 7), torch.randn(11, 7)]
    assert float(U.mtp_loss(torch.randn(2, 5, 7), heads, labels)) > 0
    pt = U.ProgressTracker(10)
    pt.update(5)
    assert pt.fraction() == 0.5 and pt.render(10).startswith("[#####.....]")


def test_training_utils_reference_verbs(tmp_path):
    s = U.MixedPrecisionScaler(64.0, interval=1)
    loss = torch.tensor(2.0)
    assert float(s.scale_loss(loss)) == 128.0 and s.current_scale() == 64.0
    good, bad = torch.nn.Parameter(torch.ones(2)), torch.nn.Parameter(torch.ones(2))
    good.grad, bad.grad = torch.ones(2), torch.tensor([1.0, float("nan")])
    assert not s.check_gradients([good]) and s.check_gradients([good, bad]) and s.check_gradients([torch.tensor([float("inf")])])
    s.update_scale(False)
    assert s.current_scale() == 128.0 and s.good_steps() == 0
    s.reset()
    assert s.current_scale() == 64.0
    w = torch.nn.Parameter(torch.tensor([1.0001, 2.0], dtype=torch.bfloat16))
    mp = U.MixedPrecisionManager(enabled=True, init_loss_scale=8.0, growth_interval=1)
    mp.create_master_weights([w])
    mp.master[0][0] = 1.0001
    assert mp.is_enabled() and mp.current_loss_scale() == 8.0 and mp.to_fp16(w).dtype == torch.bfloat16 and mp.to_fp32(mp.to_fp16(w)).dtype == torch.float32
    mp.sync_weights_to_model()
    assert float(w.data[0]) == 1.0                                       # rounded to the compute precision
    w.grad = torch.tensor([8.0, 16.0], dtype=torch.bfloat16)
    mp.cast_gradients_to_fp32()
    mp.unscale_gradients()
    assert w.grad is None and w.main_grad.dtype == torch.float32 and w.main_grad.tolist() == [1.0, 2.0] and not mp.check_gradients()
    assert mp.update_loss_scale(True) == 4.0 and float(mp.scale_loss(torch.tensor(1.0))) == 4.0
    w.data.fill_(5.0)
    mp.sync_weights_from_model()
    assert mp.master[0].tolist() == [5.0, 5.0]
    off = U.MixedPrecisionManager(enabled=False)
    assert float(off.scale_loss(torch.tensor(3.0))) == 3.0 and off.update_loss_scale(True) == 1.0
    p = torch.nn.Parameter(torch.ones(3))
    ema = U.EMAWeightAveraging(0.5).init([p])
    p.data.fill_(3.0)
    ema.update([p])
    ema.copy_to_model([p])
    assert p.data.tolist() == [2.0] * 3
    pt = U.ProgressTracker(4, log_interval=2)
    assert [pt.step() for _ in range(4)] == [False, True, False, True] and pt.is_done() and pt.current_step() == 4 and pt.total_steps() == 4
    assert pt.progress() == 1.0 and pt.elapsed_sec() >= 0 and pt.eta_sec() == 0
    pt.reset()
    assert pt.current_step() == 0
    mt = U.MetricTracker(0.5, True)
    assert mt.update(4.0) == 4.0 and mt.improved() and mt.update(2.0) == 3.0 and mt.improved() and mt.update(9.0) == 6.0 and not mt.improved()
    assert mt.best() == 3.0 and mt.value() == 6.0 and mt.steps() == 3 and mt.alpha() == 0.5
    es = U.EarlyStopping(patience=2, min_delta=0.0)
    for v in (1.0, 0.5, 0.6, 0.7):
        es.step(v)
    assert es.stopped() and es.best_epoch() == 1 and es.best_metric() == 0.5
    es.reset()
    assert not es.stopped() and es.best_metric() is None
    lw = U.LearningRateWarmup(2.0, 4)
    assert lw.get_lr(1) == 1.0 and lw.warmup_steps() == 4 and lw.target_lr() == 2.0
    a, b = torch.nn.Parameter(torch.zeros(2)), torch.nn.Parameter(torch.zeros(2))
    acc = U.GradientAccumulator(2)
    opt = torch.optim.SGD([a, b], lr=1.0)
    a.grad, b.grad = torch.tensor([1.0, 1.0]), torch.tensor([2.0, 2.0])
    assert not acc.accumulate([a, b])
    a.grad, b.grad = torch.tensor([3.0, 3.0]), torch.tensor([4.0, 4.0])
    assert acc.accumulate([a, b]) and acc.ready() and acc.current_step() == 2 and acc.accumulation_steps() == 2
    acc.apply_grads([a, b], opt)
    assert a.data.tolist() == [-2.0, -2.0] and b.data.tolist() == [-3.0, -3.0] and acc.current_step() == 0
    snap = U.ModelSnapshot(str(tmp_path / "snap.pt"))
    assert snap.load(opt, [a, b]) is None
    snap.save(opt, 7, 0.25, [a, b])
    a.data.zero_()
    assert snap.load(opt, [a, b]) == (7, 0.25) and a.data.tolist() == [-2.0, -2.0] and snap.path().endswith("snap.pt")
