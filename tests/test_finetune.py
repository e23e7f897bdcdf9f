"""LoRA / DoRA adapters (gradients vs autograd, .nrad round trip, merge), selective tuning, knowledge slots."""
import pytest
import torch

from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.trainer.finetune import (KnowledgeExpansionEngine, RankAdapterConfig, RankAdapterEngine,
                                                     SelectiveFineTuner, SelectiveTunerConfig)


def tiny(seed=0):
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, ffn_hidden_size=64, max_seq_len=32)
    return DenseModel(cfg, device="cpu", dtype=torch.float32, seed=seed)


def batch(seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 64, (2, 16), generator=g)
    return ids, torch.roll(ids, -1, 1)


@pytest.mark.parametrize("dora", [False, True])
def test_adapter_gradients_match_autograd(dora):
    m = tiny()
    eng = RankAdapterEngine(m, RankAdapterConfig(rank=4, use_dora=dora, learning_rate=0.0, warmup_steps=1))
    with torch.no_grad():
        for a in eng.adapters:
            a.B.normal_(0, 0.05)
    ids, labels = batch()
    # reference: autograd straight through the model's differentiable path with W_eff substituted
    eff = eng._materialise()
    logits = m.forward(ids)
    loss = torch.nn.functional.cross_entropy(logits.view(-1, 64), labels.reshape(-1))
    m.flat.zero_grad()
    loss.backward()                      # the block nodes leave weight gradients in .main_grad
    gW = [l.down.main_grad.clone() for l in m.layers]
    want = torch.autograd.grad(eff, [p for a in eng.adapters for p in a.params()], list(gW))
    got_loss = eng.train_step(ids, labels)
    got = [p.grad for a in eng.adapters for p in a.params()]
    assert abs(got_loss - float(loss)) < 1e-4
    for w, g in zip(want, got):
        assert torch.allclose(w, g, rtol=2e-3, atol=2e-6)


def test_lora_trains_saves_merges(tmp_path):
    m = tiny()
    base = [l.down.data.clone() for l in m.layers]
    eng = RankAdapterEngine(m, rank=4, lr=2e-2, warmup_steps=1, factor_format="q16", targets=("down", "o"))
    ids, labels = batch()
    l0 = eng.train_step(ids, labels)
    for _ in range(30):
        l1 = eng.train_step(ids, labels)
    assert l1 < l0 - 0.05
    assert eng.adapter_param_count() == 2 * (4 * 64 + 32 * 4) + 2 * (4 * 32 + 32 * 4)
    p = eng.save(tmp_path / "a.nrad")
    m2 = tiny()
    e2 = RankAdapterEngine(m2, rank=4, targets=("down", "o"))
    assert e2.load(p) and not e2.load(tmp_path / "missing.nrad")
    out1 = eng.forward_with_adapters(ids)
    out2 = e2.forward_with_adapters(ids)
    assert (out1 - out2).abs().max() < 5e-3
    eng.merge_into_base()
    assert not torch.equal(m.layers[0].down.data, base[0])
    assert torch.allclose(eng.forward_with_adapters(ids), out1, atol=1e-5)
    assert all(float(a.B.abs().max()) == 0 for a in eng.adapters)


def test_select_blocks_rule():
    g = torch.zeros(256 * 100)
    g[256 * 3: 256 * 4] = 1.0
    g[256 * 50: 256 * 51] = 0.5
    mask, thr = SelectiveFineTuner.select_blocks(g, torch.zeros_like(g), 256, 1.0, 0.5, 0.01)
    assert mask.nonzero().reshape(-1).tolist() == [3, 50] and thr > 0
    mask, _ = SelectiveFineTuner.select_blocks(torch.ones(256 * 100), torch.zeros(256 * 100), 256, 1.0, 0.5, 0.05)
    assert int(mask.sum()) == 5        # nothing exceeds mean + sigma*std: the floor applies
    f = torch.zeros_like(g)
    f[256 * 50: 256 * 51] = 100.0      # Fisher bias lifts block 50 above block 3
    mask, _ = SelectiveFineTuner.select_blocks(g, f, 256, 2.0, 0.5, 0.0)
    assert 50 in mask.nonzero().reshape(-1).tolist()


def test_selective_tuner_moves_only_selected():
    m = tiny()
    t = SelectiveFineTuner(m, SelectiveTunerConfig(learning_rate=1e-2, warmup_steps=1, ste_roundtrip=True, target_format="q16",
                                                   saliency_sigma=1.0))
    ids, labels = batch()
    t.accumulate_fisher(ids, labels)
    before = t.master.clone()
    l0 = t.fine_tune(ids, labels, 1)
    moved = (t.master != before).view(-1)
    assert 0 < t.stats.selected_fraction < 0.5
    assert moved.sum() > 0 and moved.float().mean() <= t.stats.selected_fraction + 1e-6
    for _ in range(15):
        l1 = t.fine_tune(ids, labels, 1)
    assert l1 < l0


def test_knowledge_slots(tmp_path):
    m = tiny()
    from transformers_fusion_b200.trainer.finetune import KnowledgeExpansionConfig
    k = KnowledgeExpansionEngine(m, KnowledgeExpansionConfig(learning_rate=1e-2, warmup_steps=1))
    k.add_slot("facts", 16)
    ids, labels = batch()
    base = m.forward(ids).detach()
    assert torch.allclose(k.forward_with_slots(ids), base, atol=1e-5)      # silent at initialisation
    l0 = k.train_step(ids, labels)
    for _ in range(60):
        l1 = k.train_step(ids, labels)
    assert l1 < l0 - 0.05
    logits, conf, used = k.forward_guarded(ids)
    assert logits.shape == base.shape and conf.shape == ids.shape and used.dtype == torch.bool
    k.save(tmp_path / "s.kexp")
    k2 = KnowledgeExpansionEngine(m)
    assert k2.load(tmp_path / "s.kexp") and k2.slot_count() == 1
    assert torch.allclose(k2.forward_with_slots(ids), k.forward_with_slots(ids), atol=1e-5)


def test_fine_tuner_configure_run_and_block_selection(tmp_path):
    import torch
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    from transformers_fusion_b200.trainer.finetune import FineTuner
    m = DenseModel(TransformerConfig(vocab_size=260, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=32),
                   device="cpu", dtype=torch.float32, seed=0)
    (tmp_path / "d.txt").write_text("abcabcabc " * 60)
    logs = []
    ft = FineTuner(m, lr=1e-3, fmt="q16").configure(learning_rate=5e-3, num_epochs=2, batch_size=2, seq_length=16, log_interval=1,
                                                     save_interval=3, output_path=str(tmp_path / "ft.quant"), tokenizer=ByteTokenizer(),
                                                     log=lambda step, loss: logs.append(loss))
    last = ft.fine_tune(str(tmp_path / "d.txt"))
    assert len(logs) >= 8 and last < logs[0] and (tmp_path / "ft.quant").exists()
    back = DenseModel.load(str(tmp_path / "ft.quant"))
    assert torch.allclose(back.tok_embeddings.data, m.tok_embeddings.data)
    g = torch.zeros(1024)
    g[256:512] = 1e-3
    g[700] = 1.0
    assert FineTuner.find_trainable_blocks(g, 1e-4) == [1, 2] and FineTuner.find_trainable_blocks(g, 1e-2) == []
    w = torch.randn(512)
    w0 = w.clone()
    ft.apply_quant_update(torch.ones(512), w, "q16", lr=0.5)
    from transformers_fusion_b200.quant.qat import ste_roundtrip_
    assert torch.allclose(w, w0 - 0.5, atol=2e-3) and torch.allclose(ste_roundtrip_(w.clone(), "q16"), w, atol=1e-3) and not torch.equal(w, w0 - 0.5)


def test_engine_step_counters_fisher_views_and_dora_magnitude_step():
    m = tiny()
    ids, lab = batch()
    eng = RankAdapterEngine(m, RankAdapterConfig(rank=4, use_dora=True, learning_rate=1e-3, warmup_steps=1))
    assert eng.step() == 0
    eng.train_step(ids, lab)
    assert eng.step() == 1
    a = eng.adapters[0]
    # autograd statement of the same thing: W' = m * V / |V| with V detached
    V = (a.W0 + a.B @ a.A).detach()
    mag = a.magnitude.detach().clone().requires_grad_(True)
    G = torch.randn(a.out_dim, a.in_dim)
    ((mag / V.norm(dim=1))[:, None] * V * G).sum().backward()
    before = a.magnitude.detach().clone()
    assert eng.magnitude_step([G] + [None] * (len(eng.adapters) - 1), 0.1) == 1
    assert torch.allclose(a.magnitude.detach(), before - 0.1 * mag.grad, atol=1e-6)
    assert eng.magnitude_step([torch.zeros(2, 2)], 0.1) == 0
    plain = RankAdapterEngine(m, RankAdapterConfig(rank=4, use_dora=False))
    assert plain.magnitude_step([G], 0.1) == 0
    st = SelectiveFineTuner(m)
    st.accumulate_fisher(ids, lab), st.accumulate_fisher(ids, lab)
    f = st.fisher_diag()
    assert len(f) == len(m.flat.params_list) and all(x.shape == p.shape for x, p in zip(f, m.flat.params_list))
    assert float(sum(x.sum() for x in f)) == pytest.approx(float(st.fisher.sum()) / 2, rel=1e-5)
