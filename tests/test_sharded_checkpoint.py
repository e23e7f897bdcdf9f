"""Sharded checkpoints: slices written per rank, manifest, resharding to another world size, consolidation, and the
TrainEngine round trip on one rank."""
import torch

from transformers_fusion_b200.utils import sharded_checkpoint as SC


def test_shards_reshard_and_consolidate(tmp_path):
    d = str(tmp_path / "ck")
    n, world = 5000, 4
    per = 2048
    full = torch.arange(per * world, dtype=torch.float32)
    full[n:] = 0
    m, v = full * 0.5, full * 0.25
    for r in range(world):
        SC.save_shard(d, r, world, n, r * per, (r + 1) * per, full[r * per:(r + 1) * per], m[r * per:(r + 1) * per], v[r * per:(r + 1) * per],
                      step=7)
    man = SC.read_manifest(d)
    assert man["world"] == 4 and man["step"] == 7 and len(man["shards"]) == 4 and man["has_moments"]
    assert torch.equal(SC.consolidate(d), full[:n])
    for new_world in (1, 2, 3, 8):
        parts = [SC.load_shard(d, r, new_world) for r in range(new_world)]
        cat = torch.cat([p[0] for p in parts])
        assert cat.numel() % new_world == 0 and torch.equal(cat[:n], full[:n]) and float(cat[n:].abs().sum()) == 0
        assert torch.equal(torch.cat([p[1] for p in parts])[:n], m[:n])
        assert torch.equal(torch.cat([p[2] for p in parts])[:n], v[:n])


def test_engine_roundtrip_single_rank(tmp_path):
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.trainer.engine import TrainEngine
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, ffn_hidden_size=48, max_seq_len=32, init_std=0.1)
    a = DenseModel(cfg, dtype=torch.float32, seed=1)
    ea = TrainEngine(a, lr=1e-2)
    ids = torch.randint(0, 64, (2, 16))
    for _ in range(3):
        ea.step(ids, torch.roll(ids, -1, 1))
    SC.save_engine(ea, str(tmp_path / "ck"), step=3)
    b = DenseModel(cfg, dtype=torch.float32, seed=2)
    eb = TrainEngine(b, lr=1e-2)
    assert SC.load_engine(eb, str(tmp_path / "ck")) == 3
    assert torch.equal(a.flat.params, b.flat.params)
    la, lb = ea.step(ids, torch.roll(ids, -1, 1)), eb.step(ids, torch.roll(ids, -1, 1))
    assert abs(float(la) - float(lb)) < 1e-6
    assert torch.allclose(a.flat.params, b.flat.params, atol=1e-7)      # same moments -> same next update
