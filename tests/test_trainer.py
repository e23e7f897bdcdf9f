"""Trainer API: loss decreases on a tiny model for several optimizers, checkpoint round trip (.quant +
.opt + resume state), schedules, gradient accumulation equivalence, EMA, UnifiedTrainer kinds."""
import math

import pytest
import torch

from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.trainer import schedulers as S
from transformers_fusion_b200.trainer.optimizers import OPTIMIZERS
from transformers_fusion_b200.trainer.trainer import (DataLoader, TrainConfig, Trainer, UnifiedTrainArgs, UnifiedTrainer,
                                                        unified_trainer_parse_kind)


def tiny(seed=0):
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=48, max_seq_len=32,
                            init_std=0.1)
    return DenseModel(cfg, dtype=torch.float32, seed=seed)


def data(n=4000, seed=0):
    g = torch.Generator().manual_seed(seed)
    base = torch.randint(0, 64, (16,), generator=g)
    return base.repeat(n // 16)   # periodic stream: learnable


@pytest.mark.parametrize("opt", sorted(OPTIMIZERS))
def test_every_optimizer_reduces_loss(opt):
    m = tiny()
    lr = {"sgd": 0.05, "lars": 0.5, "lion": 1e-3, "adagrad": 0.05, "adabound": 1e-2, "novograd": 0.02}.get(opt, 5e-3)
    t = Trainer(m).compile(opt, TrainConfig(batch_size=4, seq_length=16, learning_rate=lr, warmup_steps=0,
                                            lr_schedule="CONSTANT", weight_decay=0.0, zero_stage=0))
    dl = DataLoader(tokens=data(), batch_size=4, seq_length=16)
    losses = [t.train_step(*dl.next_batch()) for _ in range(40)]
    assert all(math.isfinite(x) for x in losses)
    assert min(losses[-5:]) < losses[0] - 0.05, (opt, losses[0], losses[-5:])


def test_checkpoint_roundtrip_and_resume(tmp_path):
    m = tiny()
    cfg = TrainConfig(batch_size=4, seq_length=16, learning_rate=5e-3, warmup_steps=2, max_steps=100, zero_stage=0)
    t = Trainer(m).compile("adamw", cfg)
    dl = DataLoader(tokens=data(), batch_size=4, seq_length=16)
    for _ in range(5):
        t.train_step(*dl.next_batch())
    p = str(tmp_path / "ck.quant")
    t.save_checkpoint(p, dl)
    ref = [t.train_step(*dl.next_batch()) for _ in range(3)]
    m2 = tiny(seed=9)
    t2 = Trainer(m2).compile("adamw", cfg)
    dl2 = DataLoader(tokens=data(), batch_size=4, seq_length=16)
    t2.load_checkpoint(p, dl2)
    assert t2.global_step == 5 and dl2.offset == dl.offset - 3
    got = [t2.train_step(*dl2.next_batch()) for _ in range(3)]
    assert all(abs(a - b) < 1e-4 for a, b in zip(ref, got)), (ref, got)


def test_grad_accumulation_matches_large_batch():
    ids, labels = DataLoader(tokens=data(), batch_size=8, seq_length=16).next_batch()
    outs = []
    for accum in (1, 4):
        m = tiny()
        t = Trainer(m).compile("adam", TrainConfig(batch_size=8, seq_length=16, grad_accum_steps=accum, learning_rate=1e-2,
                                                   warmup_steps=0, lr_schedule="CONSTANT", zero_stage=0, max_grad_norm=0))
        t.train_step(ids, labels)
        outs.append(m.flat.params.clone())
    assert torch.allclose(outs[0], outs[1], atol=2e-5)


def test_schedules():
    assert abs(S.schedule_lr("WARMUP_COSINE", 1.0, 0, 100, 10) - 0.1) < 1e-9
    assert abs(S.schedule_lr("WARMUP_COSINE", 1.0, 10, 100, 10) - 1.0) < 1e-9
    assert S.schedule_lr("COSINE", 1.0, 100, 100) == S.LR_FLOOR
    assert len(S.ALL) == 14
    assert abs(S.OneCycle(1.0, 100)(30) - 1.0) < 1e-6
    assert S.MultiStep(1.0, [10, 20], 0.1)(25) == pytest.approx(0.01)
    seq = S.Sequential([S.Warmup(1.0, 10), S.CosineDecay(1.0, 90)], [10])
    assert seq(5) == pytest.approx(0.6) and seq(10) == pytest.approx(1.0)
    r = S.ReduceLROnPlateau(1.0, patience=1)
    for x in (1.0, 1.0, 1.0, 1.0):
        r.observe(x)
    assert r(0) < 1.0
    assert S.Cyclic(0.1, 1.0, 10)(10) == pytest.approx(1.0)


def test_unified_trainer_and_ema(tmp_path):
    assert unified_trainer_parse_kind("ft") == "finetune" and unified_trainer_parse_kind("nope") is None
    m = tiny()
    u = UnifiedTrainer(m).configure(UnifiedTrainArgs(kind="pretrain", optimizer="adafactor", batch_size=4, seq_length=16,
                                                     lr=1e-2, output=str(tmp_path / "o.quant")))
    dl = DataLoader(tokens=data(), batch_size=4, seq_length=16)
    l0 = u.train_step_once(*dl.next_batch())
    for _ in range(30):
        l1 = u.train_step_once(*dl.next_batch())
    assert l1 < l0
    with pytest.raises(ValueError):
        UnifiedTrainer(m).configure(UnifiedTrainArgs(kind="weird"))
    u.trainer.ema_init(0.5)
    before = m.flat.params.clone()
    u.train_step_once(*dl.next_batch()); u.trainer.ema_step(); u.trainer.ema_swap()
    assert not torch.equal(m.flat.params, before)


def test_engine_gradient_accumulation_matches_full_batch():
    """Two half-batch micro-steps with grad_accum_steps=2 apply ONE update equal to a full-batch step."""
    import torch
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.trainer.engine import TrainEngine
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 64, (4, 16), generator=g)
    labels = torch.roll(ids, -1, 1)
    a = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=5)
    b = DenseModel(cfg, device="cpu", dtype=torch.float32, seed=5)
    ea = TrainEngine(a, lr=1e-2, max_grad_norm=0.0)
    eb = TrainEngine(b, lr=1e-2, max_grad_norm=0.0, grad_accum_steps=2)
    ea.step(ids, labels)
    before = b.flat.params.clone()
    eb.step(ids[:2], labels[:2])
    assert torch.equal(b.flat.params, before) and eb.opt.step_count == 0     # window still open: no update yet
    eb.step(ids[2:], labels[2:])
    assert eb.opt.step_count == 1
    assert (a.flat.params - b.flat.params).abs().max() < 1e-5


def _tiny_trainer(opt="sgd", **cfgkw):
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.trainer.trainer import TrainConfig, Trainer
    m = DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=16,
                                     init_std=0.1, **cfgkw.pop("model", {})), device="cpu", dtype=torch.float32, seed=0)
    kw = dict(batch_size=4, seq_length=16, learning_rate=5e-2, warmup_steps=0, lr_schedule="CONSTANT", max_grad_norm=0.0, zero_stage=0)
    kw.update(cfgkw)
    return Trainer(m).compile(opt, TrainConfig(**kw))


def test_qat_straight_through_absmax_and_lsq():
    import torch as T
    g = T.Generator().manual_seed(0)
    ids = T.randint(0, 64, (4, 16), generator=g)
    lab = T.roll(ids, -1, 1)
    t = _tiny_trainer(qat_bits=4)                                 # the configuration switch turns it on
    assert t.qat_enabled()
    w0 = t.model.flat.params.clone()
    l0 = t.train_step(ids, lab)
    # the weights stay unquantised (many distinct values), yet the loss was computed on 4-bit weights
    mat = t.model.layers[0].qkv.data
    assert mat.unique().numel() > 100 and not T.equal(t.model.flat.params, w0)
    q = t.qat_fake_quantize(mat)
    assert q.unique().numel() <= 15 and (q - mat).abs().max() <= mat.abs().max() / 7 / 2 + 1e-6
    plain = _tiny_trainer()
    assert abs(plain.train_step(ids, lab) - l0) > 1e-6            # the quantised forward really differs
    losses = [t.train_step(ids, lab) for _ in range(30)]
    assert losses[-1] < l0 - 0.3
    t.disable_qat()
    assert not t.qat_enabled()
    # learned step sizes: one per matrix, they move and stay positive
    t2 = _tiny_trainer()
    t2.enable_qat(4, True, use_lsq=True)
    t2.train_step(ids, lab)
    first = {i: float(s) for i, s in t2._qat_steps.items()}
    for _ in range(5):
        t2.train_step(ids, lab)
    assert first and all(float(s) > 0 for s in t2._qat_steps.values())
    assert any(abs(float(t2._qat_steps[i]) - v) > 0 for i, v in first.items())
    step = T.nn.Parameter(T.tensor([0.05]))
    y = t2.qat_fake_quantize_lsq(mat.clone().requires_grad_(True), step)
    y.sum().backward()
    assert step.grad is not None and y.unique().numel() <= 16


def test_continual_learning_consolidation_and_replay():
    import torch as T
    from transformers_fusion_b200.trainer.continual import ContinualEngineConfig
    from transformers_fusion_b200.trainer.trainer import DataLoader
    g = T.Generator().manual_seed(1)
    task_a = T.randint(0, 32, (16,), generator=g).repeat(60)
    task_b = T.randint(32, 64, (16,), generator=g).repeat(60)

    def run(continual):
        t = _tiny_trainer(learning_rate=0.1)
        if continual:
            t.enable_continual(ContinualEngineConfig(ecc_lambda=50.0, ecc_alpha=0.1, replay_capacity=64))
            t.set_replay_ratio(0.25)
            assert t.continual_enabled() and t.continual_engine() is t.continual
        dl_a, dl_b = DataLoader(tokens=task_a, batch_size=4, seq_length=16), DataLoader(tokens=task_b, batch_size=4, seq_length=16)
        for _ in range(25):
            t.train_step(*dl_a.next_batch())
        base = t.eval_loss(DataLoader(tokens=task_a, batch_size=4, seq_length=16), 2)
        got = t.on_task_boundary(1, DataLoader(tokens=task_a, batch_size=4, seq_length=16), 2)
        if continual:
            assert got == pytest.approx(base) and t._ewc_anchored and len(t._replay) > 0
        for _ in range(25):
            t.train_step(*dl_b.next_batch())
        return base, t.eval_loss(DataLoader(tokens=task_a, batch_size=4, seq_length=16), 2), t
    base_p, after_p, _ = run(False)
    base_c, after_c, tc = run(True)
    assert after_p > base_p + 0.5                                   # plain training forgets task A
    assert after_c - base_c < 0.5 * (after_p - base_p)              # consolidation + replay keep most of it
    assert any(r[2] == 0 for r in tc._replay) and tc.current_task == 1
    tc.set_ewc_lambda(3.0)
    assert tc.continual.cfg.ecc_lambda == 3.0
    tc.disable_continual()
    assert not tc.continual_enabled()


def test_loss_helpers_and_scale_rule():
    import torch as T
    from transformers_fusion_b200.trainer.trainer import Trainer
    g = T.Generator().manual_seed(2)
    logits = T.randn(2, 5, 11, generator=g)
    labels = T.randint(0, 11, (2, 5), generator=g)
    ls = Trainer.label_smoothing_loss(logits, labels, 0.1)
    want = T.nn.functional.cross_entropy(logits.view(-1, 11), labels.view(-1), label_smoothing=0.1, reduction="none").view(2, 5)
    assert T.allclose(ls, want, atol=1e-5)
    bad = labels.clone()
    bad[0, 0] = 99
    assert float(Trainer.label_smoothing_loss(logits, bad, 0.1)[0, 0]) == 0.0
    heads = [T.randn(2, 5, 11, generator=g) for _ in range(2)]
    m = Trainer.mtp_loss(heads, labels)
    w0 = T.nn.functional.cross_entropy(heads[0][:, :-1].reshape(-1, 11), labels[:, 1:].reshape(-1))
    w1 = T.nn.functional.cross_entropy(heads[1][:, :-2].reshape(-1, 11), labels[:, 2:].reshape(-1))
    assert m == pytest.approx(float(w0 + w1) / 2, rel=1e-5) and Trainer.mtp_loss([], labels) == 0.0
    t = _tiny_trainer(model=dict(mtp_num_heads=1), mtp_loss_weight=0.5)
    assert t.model.mtp_loss_weight == 0.5
    ids = T.randint(0, 64, (4, 16), generator=g)
    lab = T.roll(ids, -1, 1)
    ce = float(T.nn.functional.cross_entropy(t.model(ids).detach().view(-1, 64), lab.view(-1)))
    assert t.rdrop_loss(ids, lab, 5.0) == pytest.approx(ce, abs=1e-5)          # deterministic model: the KL term vanishes
    t.train_step(ids, lab)
    assert t.model.mtp_heads[0].main_grad is not None
    t.loss_scale, t.cfg.loss_scale_interval = 64.0, 2
    assert t.dynamic_loss_scale(5.0, 1.0) == 32.0 and t.dynamic_loss_scale(0.5, 1.0) == 32.0 and t.dynamic_loss_scale(0.5, 1.0) == 64.0
    t.loss_scale = 1.0
    assert t.dynamic_loss_scale(1e9, 1.0) == 1.0
    t.ema_init(0.5)
    t.train_step(ids, lab)
    avg = t.ema.shadow.clone()
    t.ema_apply()
    assert T.equal(t.model.flat.params, avg) and T.equal(t.ema.shadow, avg) and t.ema_enabled()


def test_dataloader_shuffle_augmentation_curriculum_and_streaming(tmp_path):
    import torch as T
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    from transformers_fusion_b200.trainer.trainer import DataLoader, ModelEMA
    from transformers_fusion_b200.utils.data import StreamingDataLoader
    dl = DataLoader(tokens=T.arange(2 * 8 * 10 + 1), batch_size=2, seq_length=8)
    assert dl.num_batches() == 10 and dl.batch_size() == 2 and dl.seq_length() == 8 and dl.has_next()
    plain = [int(dl.next_batch()[0][0, 0]) for _ in range(10)]
    assert plain == list(range(0, 160, 16)) and not dl.has_next()
    dl.shuffle(epoch=1)
    shuffled = [int(dl.next_batch_with_labels()[0][0, 0]) for _ in range(10)]
    assert sorted(shuffled) == plain and shuffled != plain
    dl.shuffle(epoch=1)
    assert [int(dl.next_batch()[0][0, 0]) for _ in range(10)] == shuffled                # same epoch, same order
    dl = DataLoader(tokens=T.arange(2 * 8 * 10 + 1), batch_size=2, seq_length=8)
    dl.set_augmentation(mask_prob=0.5, replace_prob=0.25, mask_id=999, vocab_size=50, seed=3)
    ids, lab = dl.next_batch()
    assert (ids == 999).any() and (ids != 999).any() and T.equal(lab[0], T.arange(1, 9))  # labels are untouched
    dl.set_augmentation()
    dl.set_curriculum(total_epochs=4, min_seq_length=2)
    assert dl.effective_seq_length() == 2
    _, lab = dl.next_batch()
    assert (lab[:, 2:] == -100).all() and (lab[:, :2] >= 0).all()
    dl.curriculum_step(2)
    assert dl.effective_seq_length() == 5
    dl.curriculum_step(9)
    assert dl.effective_seq_length() == 8 and (dl.next_batch()[1] >= 0).all()
    (tmp_path / "s.txt").write_text("hello streaming loader\n" * 40)
    sl = StreamingDataLoader(ByteTokenizer(), [str(tmp_path / "s.txt")], 2, 8, prefetch=2)
    first = sl.next_batch()
    assert first[0].shape == (2, 8) and sl.batch_size() == 2 and sl.seq_length() == 8 and sl.num_batches() >= 1
    n = 1
    while sl.next_batch() is not None:
        n += 1
    assert n > 3 and sl.next_batch() is None
    sl.reset()
    again = sl.next_batch()
    assert T.equal(again[0], first[0])
    sl.close()
    t = _tiny_trainer()
    ema = ModelEMA(t.model.flat, 0.5)
    t.model.flat.params.add_(1.0)
    ema.update()
    ema.set_decay(0.9)
    assert ema.decay == 0.9 and T.allclose(ema.shadow, t.model.flat.params.float() - 0.5)


def test_adamw_built_in_schedule_reset_and_scheduler_get_lr():
    from transformers_fusion_b200.trainer.optimizers import AdamW
    m = tiny()
    flat = m.flatten()
    opt = AdamW(flat, lr=1e-2, weight_decay=0.0)
    with pytest.raises(ValueError):
        opt.set_schedule("triangle")
    opt.set_schedule("warmup_cosine", warmup_steps=10, total_steps=110)
    assert opt.scheduler_step(5) == pytest.approx(5e-3) and opt.scheduler_step(10) == pytest.approx(1e-2)
    assert opt.scheduler_step(60) == pytest.approx(5e-3) and opt.scheduler_step(110) == pytest.approx(0.0, abs=1e-9)
    opt.set_schedule("linear", total_steps=100)
    assert opt.adjusted_lr(25) == pytest.approx(7.5e-3)
    opt.set_schedule("cosine_restart", total_steps=100, restart_period=20)
    assert opt.adjusted_lr(0) == pytest.approx(1e-2) and opt.adjusted_lr(20) == pytest.approx(5e-3) and opt.adjusted_lr(30) == pytest.approx(2.5e-3)
    # the scheduled rate is the one the next step uses: rate 0 leaves the weights where they are
    opt.set_schedule("linear", total_steps=10)
    opt.scheduler_step(10)
    before = flat.params.clone()
    flat.grads.fill_(1.0)
    opt.step()
    assert torch.equal(flat.params, before) and opt.step_count == 1
    opt.scheduler_step(0)
    flat.grads.fill_(1.0)
    opt.step()
    assert not torch.equal(flat.params, before) and "m" in opt.state
    opt.reset()
    assert opt.state == {} and opt.step_count == 0 and opt.current_lr is None and torch.equal(opt.master, flat.params.float()) and opt.get_lr() == 1e-2
    sch = S.LinearWarmupDecay(1.0, 10, 110)
    assert sch.get_last_lr() == 1.0 and sch.get_lr(5) == pytest.approx(sch(5)) and sch.get_last_lr() == pytest.approx(sch(5))
    assert S.CosineWarmupRestart(1.0, 0, 10).get_lr(5) == pytest.approx(S.CosineWarmupRestart(1.0, 0, 10)(5))


def test_unified_trainer_inner_and_mixed_precision_restart():
    m = tiny()
    u = UnifiedTrainer(m)
    assert u.inner() is None
    with pytest.raises(RuntimeError):
        u.set_log_callback(print)
    u.configure(UnifiedTrainArgs(kind="dense", optimizer="adamw", batch_size=2, seq_length=16, lr=1e-3))
    t = u.inner()
    assert isinstance(t, Trainer)
    cb = lambda *a: None
    u.set_log_callback(cb)
    assert t.log_cb is cb
    m.flat.params.add_(1.0)                                    # weights changed behind the optimizer's back
    assert t.init_mixed_precision() == 1.0 and torch.equal(t.opt.master, m.flat.params[t.opt.lo:t.opt.hi].float())
    t.cfg.dynamic_loss_scale, t.loss_scale = True, 4.0
    assert t.init_mixed_precision() == t.cfg.loss_scale
