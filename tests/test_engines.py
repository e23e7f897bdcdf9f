"""Engine facades and host planners: ring all-reduce oracle, TP splits, shard / pipeline plans, losses with explicit
gradients against autograd, optimiser suite, loaders, bare checkpoints, policy-gradient helpers, MoE routing / dispatch
oracles against the dense weighted sum, DenseTrainer / MoETrainerEngine bookkeeping, text facade with stream buffering."""
import math

import pytest
import torch

from transformers_fusion_b200.engines import dense as D, inference as I, moe as ME, parallel as P
from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.trainer.trainer import TrainConfig


def tiny(seed=0, **kw):
    base = dict(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=48, max_seq_len=64, init_std=0.1)
    base.update(kw)
    return DenseModel(TransformerConfig(**base), dtype=torch.float32, seed=seed)


def stream(n=4000, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 64, (16,), generator=g).repeat(n // 16)


# ------------------------------------------------------------------------------------------------ parallel planners
@pytest.mark.parametrize("world,n", [(2, 10), (3, 17), (4, 64), (5, 3)])
def test_ring_allreduce_equals_sum(world, n):
    g = torch.Generator().manual_seed(world * 100 + n)
    bufs = [torch.randn(n, generator=g) for _ in range(world)]
    want = torch.stack(bufs).sum(0)
    P.ring_allreduce_sum(bufs)
    for b in bufs:
        assert torch.allclose(b, want, atol=1e-5)


def test_slices_tp_splits_and_plans():
    sl = [P.slice_for(10, r, 4) for r in range(4)]
    assert [s.count for s in sl] == [3, 3, 2, 2] and [s.start for s in sl] == [0, 3, 6, 8]
    w = torch.arange(48.).view(8, 6)
    assert torch.equal(P.tp_gather_cols(P.tp_split_cols(w, 4).shards), w)
    assert torch.equal(P.tp_gather_rows(P.tp_split_rows(w, 3).shards), w)
    x = torch.randn(5, 6)
    # column-parallel: concatenated outputs; row-parallel: summed partial outputs
    assert torch.allclose(torch.cat([x @ s.t() for s in P.tp_split_cols(w, 2).shards], 1), x @ w.t())
    parts = [x[:, i * 2:(i + 1) * 2] @ s.t() for i, s in enumerate(P.tp_split_rows(w, 3).shards)]
    assert torch.allclose(sum(parts), x @ w.t(), atol=1e-4)
    bufs = [torch.full((4,), float(r)) for r in range(3)]
    P.broadcast_bufs(bufs, 2)
    assert all(torch.equal(b, torch.full((4,), 2.0)) for b in bufs)
    sp = P.plan_shards(["a", "b", "c", "d"], [100, 10, 10, 80], 2)
    assert sp.rank_bytes == [400, 400] and sp.total_bytes == 800 and sp.imbalance() == 0.0
    pp = P.plan_pipeline(10, 4)
    assert pp.stage_layers == [3, 2, 3, 2] and pp.layer_stage[0] == 0 and pp.layer_stage[-1] == 3
    with pytest.raises(ValueError):
        P.plan_pipeline(0, 2)


# ------------------------------------------------------------------------------------------------ losses
def _auto_grad(fn, logits):
    lg = logits.clone().requires_grad_(True)
    loss = fn(lg)
    return float(loss.detach()), torch.autograd.grad(loss, lg)[0]


def test_losses_match_autograd():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(12, 9, generator=g)
    labels = torch.randint(0, 9, (12,), generator=g)
    labels[3] = -100
    TF = torch.nn.functional
    out, d = D.ce_loss(logits, labels)
    l, dg = _auto_grad(lambda x: TF.cross_entropy(x, labels, ignore_index=-100), logits)
    assert abs(out.loss - l) < 1e-5 and torch.allclose(d, dg, atol=1e-6) and 0 <= out.acc <= 1
    out, d = D.label_smooth_ce(logits, labels, 0.1)
    l, dg = _auto_grad(lambda x: TF.cross_entropy(x, labels, ignore_index=-100, label_smoothing=0.1), logits)
    assert abs(out.loss - l) < 1e-5 and torch.allclose(d, dg, atol=1e-6)
    out, d = D.focal_loss(logits, labels, gamma=0.0, alpha=1.0)          # gamma 0, alpha 1 -> plain CE
    assert abs(out.loss - D.ce_loss(logits, labels)[0].loss) < 1e-5
    out2, _ = D.focal_loss(logits, labels, gamma=2.0, alpha=0.25)
    assert out2.loss < 0.25 * out.loss + 1e-6
    adv = torch.randn(12, generator=g)
    l, d = D.policy_grad_loss(logits, labels, adv)
    keep = labels != -100
    ref = lambda x: -(adv * torch.log_softmax(x, -1).gather(1, labels.clamp(min=0)[:, None])[:, 0] * keep).sum() / keep.sum()
    l2, dg = _auto_grad(ref, logits)
    assert abs(l - l2) < 1e-5 and torch.allclose(d, dg, atol=1e-6)
    pred, tgt = torch.randn(4, 5, generator=g), torch.randn(4, 5, generator=g)
    out, d = D.mse_loss_fn(pred, tgt)
    _, dg = _auto_grad(lambda x: ((x - tgt) ** 2).mean(), pred)
    assert torch.allclose(d, dg, atol=1e-6)
    r = D.rdrop_loss(logits, logits, labels)
    assert r.kl < 1e-6 and abs(r.total - r.ce) < 1e-6
    loss, da, db = D.infonce_loss(torch.randn(6, 8, generator=g), torch.randn(6, 8, generator=g))
    assert loss > 0 and da.shape == (6, 8) and db.shape == (6, 8)
    assert D.seq_z_loss(torch.zeros(3, 4)) == pytest.approx(math.log(4) ** 2, rel=1e-5)


def test_grpo_and_reward_normalisation():
    g = torch.Generator().manual_seed(1)
    logits, labels = torch.randn(8, 5, 11, generator=g), torch.randint(0, 11, (8, 5), generator=g)
    rewards = torch.tensor([1., 0, 0, 1, 2, 2, 2, 2])
    out = D.grpo_step(logits, labels, rewards, group=4)
    assert out.mean_reward == pytest.approx(1.25) and math.isfinite(out.loss)
    # ratio 1 and standardised advantages: the surrogate is -mean(adv) = 0 for the mixed group and 0 for the constant one
    assert abs(out.loss) < 1e-5
    st = D.normalize_rewards(rewards)
    assert st.mean == pytest.approx(1.25) and st.std > 0
    with pytest.raises(ValueError):
        D.grpo_step(logits, labels, rewards, group=3)


# ------------------------------------------------------------------------------------------------ optimiser suite / schedule
@pytest.mark.parametrize("kind", D.OptimSuite.KINDS)
def test_optim_suite_descends_quadratic(kind):
    torch.manual_seed(0)
    a, b = torch.randn(6, 4), torch.randn(5)
    ta, tb = torch.ones(6, 4), torch.zeros(5)
    suite = D.OptimSuite(kind, lr={"sgd": 0.1, "lion": 0.03, "adafactor": 0.05}.get(kind, 0.05), wd=0.0)
    suite.add_group([a], 1.0, 1.0)
    suite.add_group([b], 0.5, 0.0)
    suite.set_schedule("CONSTANT", 0, 100)
    first = None
    for step in range(120):
        a.grad, b.grad = 2 * (a - ta), 2 * (b - tb)
        loss = float(((a - ta) ** 2).sum() + ((b - tb) ** 2).sum())
        first = loss if first is None else first
        suite.scheduler_step(step)
        suite.clip(10.0)
        suite.step()
        suite.zero_grad()
    assert loss < 0.2 * first, (kind, first, loss)
    assert suite.stats().steps == 120 and suite.stats().last_update_norm >= 0
    snap = D.OptimSuite.snapshot([a])
    a.add_(1.0)
    assert D.OptimSuite.update_norm(snap, [a]) == pytest.approx(math.sqrt(24), rel=1e-5)


def test_lr_schedule_shape():
    s = D.LRSchedule("WARMUP_COSINE", 1.0, 10, 100, 0.1)
    assert s.lr_at(0) < s.lr_at(5) < s.lr_at(10) and s.lr_at(10) == pytest.approx(1.0, rel=1e-2)
    assert s.lr_at(100) == pytest.approx(0.1, rel=1e-2)


# ------------------------------------------------------------------------------------------------ data
class _CharTok:
    eos_id = 0

    def encode(self, s): return [ord(c) % 64 for c in s]
    def decode(self, ids): return "".join(chr(97 + i % 26) for i in ids)


def test_loaders_augment_curriculum(tmp_path):
    p = tmp_path / "t.txt"
    p.write_text("hello world, this is a tiny corpus. " * 60)
    tok = _CharTok()
    dl = D.DenseDataLoader(tok, str(p), 2, 8)
    a, b = dl.next_batch()
    assert a.shape == (2, 8) and torch.equal(a.reshape(-1)[1:], b.reshape(-1)[:-1])
    dl.shuffle(1)
    a1, b1 = dl.next_batch()
    assert torch.equal(a1[:, 1:], b1[:, :-1]) and dl.num_batches() > 10
    dl.shuffle(1)
    assert torch.equal(dl.next_batch()[0], a1)                       # same epoch seed, same order
    sd = D.StreamDataLoader(tok, str(p), 2, 8, chunk_bytes=64)
    seen = []
    while (bt := sd.next_batch()) is not None:
        seen.append(bt[0].reshape(-1))
    sd.close()
    full = torch.tensor(tok.encode(p.read_text()))
    got = torch.cat(seen)
    assert torch.equal(got, full[:got.numel()]) and sd.batches_served() == len(seen) > 5
    pol = D.AugmentPolicy(token_dropout=0.5, span_mask_prob=0.3, span_len=4, pad_id=63, seed=7)
    ids = torch.zeros(4, 64, dtype=torch.long)
    pol.apply_ids(ids)
    frac = float((ids == 63).float().mean())
    assert 0.4 < frac < 0.9
    lg = torch.zeros(8, 8)
    D.AugmentPolicy(logit_noise_std=0.1).apply_logits(lg)
    assert 0.03 < float(lg.std()) < 0.3
    c = D.Curriculum(64, 512, 3, 0)
    assert c.effective_len() == 64 and D.Curriculum(64, 512, 3, 2).effective_len() == 512
    assert D.Curriculum(64, 512, 4, 1).difficulty_mix() == 0.5


def test_dense_checkpoint_roundtrip(tmp_path):
    ps = [torch.randn(3, 4), torch.randn(7)]
    path = str(tmp_path / "p.tfdc")
    D.DenseCheckpoint.save(path, ps, 123)
    qs = [torch.zeros(3, 4), torch.zeros(7)]
    assert D.DenseCheckpoint.load(path, qs) == 123
    assert all(torch.equal(a, b) for a, b in zip(ps, qs))
    with pytest.raises(ValueError):
        D.DenseCheckpoint.load(path, [torch.zeros(3, 4)])


# ------------------------------------------------------------------------------------------------ trainers
def test_dense_trainer_facade_tracks_stats(tmp_path):
    from transformers_fusion_b200.trainer.trainer import DataLoader
    m = tiny()
    t = D.DenseTrainer(m).compile("adamw", TrainConfig(batch_size=4, seq_length=16, learning_rate=5e-3, warmup_steps=0,
                                                       lr_schedule="CONSTANT", weight_decay=0.0, zero_stage=0))
    dl = DataLoader(tokens=stream(), batch_size=4, seq_length=16)
    losses = [t.train_step(*dl.next_batch()) for _ in range(30)]
    s = t.stats()
    assert s.steps == 30 and s.tokens == 30 * 64 and s.tok_per_sec > 0 and s.last_loss == pytest.approx(losses[-1])
    assert losses[-1] < losses[0] - 0.05
    v = t.eval_loss(DataLoader(tokens=stream(), batch_size=4, seq_length=16), 3)
    assert s.best_val_loss == pytest.approx(v) and s.eval_batches == 3
    ev = D.eval_loop(t.trainer, DataLoader(tokens=stream(), batch_size=4, seq_length=16), 2)
    assert ev.batches == 2 and ev.perplexity == pytest.approx(math.exp(ev.loss), rel=1e-4)
    t.save_checkpoint(str(tmp_path / "m.quant"))
    u = D.UnifiedEntry(tiny(), None)
    ok, err = u.configure(D.UnifiedTrainArgs(kind="nonsense"))
    assert not ok and "nonsense" in err
    ok, err = u.configure(D.UnifiedTrainArgs(kind="dense", optimizer="adamw", batch_size=4, seq_length=16, lr=1e-3))
    assert ok, err
    ok, loss, err = u.train_step_once(*dl.next_batch())
    assert ok and math.isfinite(loss) and u.stats().steps == 1
    assert D.UnifiedEntry.parse_kind("moe") == "moe" and D.UnifiedEntry.kind_name("??") == "unknown"


def test_eval_harness_and_ngrams():
    m = tiny()
    h = D.EvalHarness(m)
    out = h.run_tokens(stream(400).tolist(), context=32)
    assert out.tokens == 400 and out.perplexity.perplexity > 1 and 0 <= out.accuracy.accuracy <= 1
    assert D.NgramScore.precision([1, 2, 3, 4], [1, 2, 3, 5], 2) == pytest.approx(2 / 3)
    assert D.NgramScore.lcs_len([1, 2, 3, 4, 5], [2, 4, 5, 6]) == 3
    assert h.bleu([1, 2, 3, 4, 5], [1, 2, 3, 4, 5]) == pytest.approx(1.0)
    assert h.rouge_l([1, 2, 3], [1, 2, 3]) == pytest.approx(1.0)
    res = h.hellaswag([[1, 2, 3]] * 3, [[4, 5]] * 3, [[6, 7]] * 3)
    assert res.total == 3 and res.accuracy in (0.0, 1.0)


# ------------------------------------------------------------------------------------------------ MoE planners
def test_moe_routing_and_dispatch_oracles():
    g = torch.Generator().manual_seed(3)
    T, E, k, Dm = 40, 8, 2, 16
    logits, hidden = torch.randn(T, E, generator=g), torch.randn(T, Dm, generator=g)
    ro = ME.route_topk(logits, k, 0.01)
    assert torch.allclose(ro.weights.sum(-1), torch.ones(T)) and ro.aux_loss > 0
    uniform = ME.route_topk(torch.zeros(T, E), 1, 1.0)
    assert uniform.aux_loss == pytest.approx(1.0, rel=1e-5)            # E * sum f_e / E with sum f_e = 1
    cp = ME.plan_capacity(T, E, k, 1.0)
    assert cp.slots_per_expert == 10 and cp.dropped == 0 and ME.plan_capacity(100, 4, 2, 0.5).dropped == 100
    experts = [torch.randn(Dm, Dm, generator=g) for _ in range(E)]
    plan = ME.plan_dispatch(ro.indices, ro.weights, E, 0)               # unlimited: equals the dense weighted sum
    xin = ME.gather_expert_inputs(hidden, plan, E)
    assert sum(xin.counts) == T * k
    out = ME.combine_expert_outputs([xin.bufs[e] @ experts[e] for e in range(E)], plan, T, Dm)
    want = torch.zeros(T, Dm)
    for t in range(T):
        for j in range(k):
            want[t] += ro.weights[t, j] * (hidden[t] @ experts[int(ro.indices[t, j])])
    assert torch.allclose(out.hidden, want, atol=1e-4) and out.dropped == 0
    tight = ME.plan_dispatch(ro.indices, ro.weights, E, 4)
    ds = ME.drop_stats(tight, E)
    assert ds.assigned == T * k and max(ds.per_expert_kept) <= 4 and ds.dropped == ds.assigned - ds.kept > 0
    assert ds.drop_rate == pytest.approx(ds.dropped / ds.assigned)
    m = ME.build_ep_map(8, 4)
    assert m.expert_rank == [0, 0, 1, 1, 2, 2, 3, 3] and m.rank_counts == [2, 2, 2, 2]
    assert ME.build_ep_map(6, 4, contiguous=False).expert_rank == [0, 1, 2, 3, 0, 1]
    b = ME.balance_stats([10, 10, 10, 10], 40)
    assert b.cv == 0 and b.min_share == 0.25 and b.max_share == 0.25
    assert ME.z_loss(torch.zeros(5, 4)) == pytest.approx(math.log(4) ** 2, rel=1e-5)


def test_moe_trainer_engine_and_pipeline(tmp_path):
    from transformers_fusion_b200.models.moe import MoEModel
    from transformers_fusion_b200.models.config import MoEConfig
    cfg = MoEConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=48, max_seq_len=64, init_std=0.1,
                    num_experts=4, top_k=2)
    m = MoEModel(cfg, dtype=torch.float32, seed=0)
    eng = ME.MoETrainerEngine(m).compile("adamw", ME.MoETrainConfig(batch_size=2, seq_length=16, learning_rate=3e-3, warmup_steps=0,
                                                                   lr_schedule="CONSTANT", max_steps=6, epochs=2))
    p = tmp_path / "train.txt"
    p.write_text("abcdefgh" * 200)
    pipe = ME.MoEPipeline(eng, _CharTok(), str(p), str(p))
    pipe.set_checkpoint_dir(str(tmp_path / "ck"))
    pipe.set_log_file(str(tmp_path / "log.jsonl"))
    last = pipe.run(2)
    assert math.isfinite(last) and pipe.best_val() < 1e30
    assert (tmp_path / "ck" / "best.quant").exists() and (tmp_path / "ck" / "epoch1.quant").exists()
    assert len((tmp_path / "log.jsonl").read_text().strip().splitlines()) == 2
    s = eng.stats()
    assert s.steps == 12 and 0 <= s.expert_util <= 1


# ------------------------------------------------------------------------------------------------ inference facade
def test_stream_buffer_and_text_facade():
    sb, got = I.StreamBuffer(), []
    for piece in ["Hel", "lo", " ", "wor", "ld", "!"]:
        sb.append(piece)
        if sb.should_flush():
            sb.flush(got.append)
    sb.flush(got.append)
    assert got == ["Hello ", "world!"]
    m = tiny(vocab_size=256, hidden_size=64, max_seq_len=128)
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    from transformers_fusion_b200.inference.sampler import SamplerConfig
    eng = I.InferenceEngine().init(m, ByteTokenizer(), I.EngineConfig(max_seq_len=128, max_tokens=12,
                                                                      sampler=SamplerConfig(temperature=0.0, top_k=0, top_p=1.0)))
    text, st = eng.generate_with_stats("abc")
    assert st.tokens_generated > 0 and st.tokens_per_sec > 0 and 0 <= st.kv_cache_utilization <= 1
    pieces = []
    eng.generate_stream("abc", pieces.append)
    assert "".join(pieces) == text
    assert eng.generate_batch(["abc", "abc"]) == [text, text]
    eng.reset_context()
    assert I.InferenceEngine().generate("x") == ""
    ok, err = I.InferenceEngine().load("/nonexistent/model.quant")
    assert not ok and "no such file" in err
