import math

import pytest
import torch

from transformers_fusion_b200.trainer import continual as C
from transformers_fusion_b200.trainer import hpo_nas as H


def objective(c, budget=1.0):
    # best at lr = 1e-3, weight_decay = 1e-2; more budget = less noise
    return -((math.log10(c.lr) + 3) ** 2 + 0.3 * (math.log10(c.weight_decay) + 2) ** 2)


def test_hpo_methods(tmp_path):
    for method, n in (("random", 40), ("bayes", 25), ("pbt", 40), ("sha", 27)):
        e = H.HPOEngine(objective, seed=1)
        best = e.optimize(n, method)
        assert abs(math.log10(best.lr) + 3) < 1.0, (method, best.lr)
        assert e.get_top_k(3)[0].id == best.id and len(e.get_eval_history()) >= min(n, 20)
    assert e.save_best_configs(str(tmp_path / "b.json"), 3)
    loaded = H.HPOEngine.load_configs(str(tmp_path / "b.json"))
    assert len(loaded) == 3 and loaded[0].lr == e.get_top_k(1)[0].lr
    plan = H.HPOEngine().setup_successive_halving(27, 5)
    assert plan.configs_per_rung == [27, 9, 3, 1] and plan.budget_per_rung == [1.0, 3.0, 9.0, 27.0]
    # the surrogate interpolates what it has seen
    e = H.HPOEngine(objective, seed=2)
    cs = e.random_search(15)
    assert abs(e.surrogate_predict(cs[0]) - cs[0].score) < 0.2


def test_nas_respects_constraints():
    hw = H.HardwareConstraints(max_params=60_000_000, enabled=True)
    nas = H.NASEngine(lambda a: math.log10(a.param_count), H.NASConfig(population=12, generations=8), hw, seed=3)
    best = nas.search()
    assert best.param_count <= 1.3 * hw.max_params and best.param_count > 5_000_000     # grows up to the limit, not past it
    a = nas.random_architecture()
    b = nas.mutate(a, H.NASMutateOp.ADD_LAYER)
    assert b.num_layers == a.num_layers + 1 and b.param_count > a.param_count and b.id != a.id
    c = nas.mutate(a, H.NASMutateOp.CHANGE_HEADS)
    assert c.hidden_size % c.num_heads == 0
    cfg = nas.to_transformer_config(best)
    assert cfg.hidden_size == best.hidden_size and cfg.num_layers == best.num_layers


def test_replay_and_ecc():
    buf = C.CompressedReplayBuffer(capacity=10, spill_threshold=0.5)
    for i in range(12):
        buf.insert(torch.full((8,), float(i)), torch.arange(8.0), task_id=i % 2, fisher_importance=float(i + 1))
    assert buf.size() <= 10 and min(e.fisher_importance for e in buf.entries) >= 6     # low-importance entries were dropped
    ins, tgs, ws = buf.sample_batch(4)
    assert len(ins) == 4 and torch.allclose(tgs[0], torch.arange(8.0), atol=0.02) and abs(sum(ws) / 4 - 1) < 1e-6
    assert buf.compression_ratio() > 1.3           # 8-element samples: the 32-byte entry header dominates; long samples approach 4x
    ecc = C.ECCState()
    ecc.initialize(4)
    ecc.update_anchor(torch.zeros(4))
    ecc.update_fisher(torch.tensor([1.0, 0.0, 2.0, 0.0]), 1.0)
    w = torch.ones(4)
    assert ecc.regularize(w, 2.0) == pytest.approx(5.0) and ecc.penalty_grad(w, 2.0).tolist() == [2.0, 0.0, 8.0, 0.0]


def test_engine_lr_governor_and_metrics():
    eng = C.ContinualEngine(C.ContinualEngineConfig(forgetting_threshold=0.1))
    w = torch.zeros(6)
    assert eng.on_step(torch.ones(6), w, 1e-3, 0) == 1e-3
    eng.on_task_boundary(1, w, baseline_loss=1.0, untrained_loss=3.0)
    eng.register_eval(0, 1.5)                                  # task 0 got worse by 0.5 > threshold
    assert eng.effective_lr(1e-3) == pytest.approx(5e-4)
    m = eng.forgetting_metrics()
    assert m.avg_forgetting == pytest.approx(0.5) and m.backward_transfer == pytest.approx(-0.5) and m.forward_transfer == pytest.approx(2.0)
    eng.register_eval(0, 1.0)
    assert eng.effective_lr(1e-3) == pytest.approx(2e-3)       # nothing forgotten: more plasticity
    g = eng.regularized_grads(torch.zeros(6), torch.ones(6))
    assert float(g.sum()) > 0


def test_projection_watchdog_entropy():
    w = torch.tensor([1.0, 0.0, 0.0])
    u = torch.tensor([0.5, 0.2, -0.1])
    C.apply_orthogonal_projection(u, w)
    assert abs(float(u @ w)) < 1e-7 and u[1] == pytest.approx(0.2)
    wd = C.DistributionWatchdog(2.0)
    layer = torch.nn.Parameter(torch.randn(1000))
    wd.track_layer(0, layer)
    good = layer.detach().clone()
    layer.data.mul_(5.0)
    wd.track_layer(0, layer)
    assert not wd.check_health()[0].is_healthy
    wd.rollback(0, layer)
    assert torch.equal(layer.data, good)
    x = torch.zeros(100)
    assert not C.apply_entropy_floor(2.0, x, torch.rand(100))
    x = torch.randn(100)
    y = x.clone()
    assert C.apply_entropy_floor(0.1, y, torch.arange(100.0), generator=torch.Generator().manual_seed(0))
    assert (y != x).sum() > 30 and torch.equal(y[60:], x[60:])
    rb = C.ExperienceReplayBuffer(3, 2)
    for i in range(5):
        rb.add(i, -i)
    assert rb.size() == 3 and rb.should_replay(4) and not rb.should_replay(3) and len(rb.sample_batch(2)[0]) == 2


def test_nas_engine_reference_verbs(tmp_path):
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.trainer.hpo_nas import Architecture, HardwareConstraints, NASConfig, NASEngine
    target = 24 * 1024 * 1024
    fit = lambda a: -abs(math.log(a.param_count / target))                # best: about 24 M parameters
    nas = NASEngine(fit, seed=3)
    nas.set_search_config(NASConfig(population=10, generations=6))
    nas.set_hardware_constraints(HardwareConstraints(enabled=True, max_params=10**9, target_memory_bytes=10**10, target_latency_ms=1e6))

    class M:
        cfg = TransformerConfig(vocab_size=1000, hidden_size=256, num_layers=4, num_heads=4, ffn_hidden_size=512, max_seq_len=64)
    nas.set_model(M())
    pop = nas.initialize_population(5)
    assert len(pop) == 5 and (pop[0].hidden_size, pop[0].num_layers) == (256, 4)
    a = pop[0]
    assert nas.mutate_add_layer(a).num_layers == 5 and nas.mutate_remove_layer(a).num_layers == 3 and nas.mutate_change_ffn(a).ffn_size != 512
    assert nas.mutate_change_width(a).hidden_size != 256 and nas.mutate_change_heads(a).num_heads != 4 and nas.mutate_change_dropout(a).dropout != a.dropout
    child = nas.crossover(pop[0], pop[1])
    assert child.num_layers in (pop[0].num_layers, pop[1].num_layers) and child.hidden_size % child.num_heads == 0
    for x in pop:
        nas.evaluate(x)
    assert nas.tournament_select(pop, 5) is max(pop, key=lambda x: x.score)
    best = nas.search(population=10, generations=6)
    assert best is nas.get_best_architecture() and abs(math.log(best.param_count / target)) < abs(math.log(pop[0].param_count / target))
    front = nas.get_pareto_front()
    assert front and front[0].score == best.score and all(f.score >= -10 for f in front)
    assert nas.save_architectures(str(tmp_path / "a.json"), 3)
    loaded = NASEngine.load_architectures(str(tmp_path / "a.json"))
    assert len(loaded) == 3 and loaded[0].score == best.score and isinstance(loaded[0], Architecture)
    assert nas.estimate_memory(4, 256, 512, 1000) == pop[0].memory_bytes and nas.estimate_latency_cycles(4, 256, 4) > 0
    small, huge = nas.hardware_aware_score(pop[0]), None
    nas.set_hardware_constraints(HardwareConstraints(enabled=True, max_params=1000, target_memory_bytes=10**10, target_latency_ms=1e6))
    assert nas.hardware_aware_score(pop[0]) < small
    nas2 = NASEngine(fit, seed=5)
    d = nas2.darts_search(30)
    first = nas2.history[0]
    assert d.score >= first.score and nas2.darts_migrate(first, 1.0).num_layers == d.num_layers
    n = len(nas2.history)
    nas2.record_architecture(first)
    assert len(nas2.history) == n + 1


def test_forgetting_benchmark_task_registry_and_transfer():
    from transformers_fusion_b200.trainer.continual import ForgettingBenchmark
    fb = ForgettingBenchmark()
    a = fb.register_task([1.0, 2.0, 3.0], [2.0, 4.0, 6.0], 2)
    b = fb.register_task([5.0], [6.0])
    assert (a, b) == (0, 1) and fb.num_tasks() == 2 and fb.eval_set(0) == ([1.0, 2.0], [2.0, 4.0])
    fb.record_current(1, 3.0)                        # task 1 measured before it was trained: the untrained loss
    fb.record_baseline(0, 1.0), fb.record_baseline(1, 1.5)
    fb.record_current(0, 1.4), fb.record_current(1, 1.5)
    assert fb.forgetting(0) == pytest.approx(0.4) and fb.forgetting(1) == 0.0 and fb.forgetting(9) == 0.0
    assert fb.backward_transfer() == pytest.approx(-0.2) and fb.forward_transfer() == pytest.approx((0.0 + 1.5) / 2)
    m = fb.compute()
    assert m.num_tasks == 2 and m.max_forgetting == pytest.approx(0.4) and m.avg_forgetting == pytest.approx(0.2)


def test_hpo_built_in_training_objective_restores_the_trainer():
    import torch
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.trainer.hpo_nas import HPConfig, HPOEngine
    from transformers_fusion_b200.trainer.trainer import DataLoader, TrainConfig, Trainer
    m = DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=48, max_seq_len=32, init_std=0.1),
                   dtype=torch.float32, seed=0)
    t = Trainer(m).compile("adamw", TrainConfig(batch_size=4, seq_length=16, learning_rate=1e-3, warmup_steps=0, lr_schedule="CONSTANT", zero_stage=0))
    base = torch.randint(0, 64, (16,), generator=torch.Generator().manual_seed(0))
    dl = DataLoader(tokens=base.repeat(100), batch_size=4, seq_length=16)
    h = HPOEngine(seed=0)
    h.set_model(m)
    h.set_trainer(t, dl, steps_per_budget=10)
    w0 = m.flat.params.clone()
    good = h._train_objective(HPConfig(id=0, lr=1e-2, weight_decay=0.0, warmup_steps=0), 2.0)
    idle = h._train_objective(HPConfig(id=1, lr=1e-9, weight_decay=0.0, warmup_steps=0), 2.0)
    assert good > idle                                            # a useful learning rate reaches a lower loss in 20 steps
    assert torch.equal(m.flat.params, w0) and t.global_step == 0 and t.cfg.learning_rate == 1e-3 and t.opt.step_count == 0
    assert h.evaluate_fn == h._train_objective
