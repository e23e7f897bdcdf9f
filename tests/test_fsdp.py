import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(n, backend, tmp_path, env):
    port = 29600 + (os.getpid() % 90) + (5 if backend == "nccl" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "_mp_fsdp_worker.py"), str(tmp_path), backend]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, **env))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return [json.load(open(os.path.join(tmp_path, f"rank{i}.json"))) for i in range(n)]


def test_zero3_matches_single_process_gloo(tmp_path):
    for res in _launch(2, "gloo", tmp_path, {"CUDA_VISIBLE_DEVICES": ""}):
        assert res["n_sharded"] >= 8 and res["savings"] > 0.3 and res["gathers"] > 20
        for a, b in zip(res["losses"], res["ref_losses"]):
            assert abs(a - b) < 2e-4, res
        assert res["param_err"] < 2e-4, res


@pytest.mark.gpu
@pytest.mark.multigpu
def test_zero3_fused_weight_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for res in _launch(2, "nccl", tmp_path, {"NCCL_NVLS_ENABLE": "0"}):
        assert res["status"] == 0, res
        for a, b in zip(res["losses"], res["ref_losses"]):
            assert abs(a - b) < 5e-2, res
        assert res["param_err"] < 5e-2, res
        assert res["losses"][-1] < res["losses"][0]


def test_offload_and_checkpointing_helpers():
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.parallel.fsdp import ActivationCheckpointing, CPUOffloadEngine, FullyShardedDataParallel
    eng = CPUOffloadEngine(pool_bytes=1 << 20, device="cpu")
    t = torch.arange(1000.0)
    eng.offload("m", t)
    assert torch.equal(eng.fetch("m"), t)
    with pytest.raises(MemoryError):
        eng.offload("big", torch.zeros(1 << 20))
    eng.release("m")
    assert eng.used == 0
    m = DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=3, num_heads=4, ffn_hidden_size=64, max_seq_len=16),
                   device="cpu", dtype=torch.float32, seed=0)
    ac = ActivationCheckpointing(m).enable()
    assert m.activation_checkpointing and ac.memory_saved_bytes(2, 16) > 0
    assert FullyShardedDataParallel.auto_wrap(m, 1000) == ["layers.0", "layers.1", "layers.2"]


def test_facade_two_call_form_precision_helpers_and_shard_optimizer(capsys):
    """forward(); backward() equals train_step's gradients; flat shard view, memory print, per-block accounting, the
    explicit save_input / recompute form and the per-shard optimizer (plain and with an fp32 master)."""
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.parallel.collectives import DistributedContext
    from transformers_fusion_b200.parallel.fsdp import (ActivationCheckpointing, FSDPBlock, FSDPConfig,
                                                       FullyShardedDataParallel, ZeROOptimizer)
    cfg = TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, ffn_hidden_size=64, max_seq_len=16)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(1))
    lab = torch.roll(ids, -1, 1)

    def make():
        f = FullyShardedDataParallel(DenseModel(cfg, device="cpu", dtype=torch.float32, seed=0),
                                     FSDPConfig(lr=1e-2, weight_decay=0.0), DistributedContext(0, 1))
        f.engine.mesh.world_group = None
        return f
    a, b = make(), make()
    logits = a.forward(ids, lab)
    assert logits.shape == (2, 16, 64)
    la = a.backward()
    a.optimizer_step()
    lb = b.train_step(ids, lab)
    assert float(la) == pytest.approx(float(lb), abs=1e-6)
    assert torch.allclose(a.flatten_and_shard(), b.flatten_and_shard(), atol=1e-6)
    with pytest.raises(RuntimeError):
        a.backward()                                                   # the batch was consumed
    assert a.stage() == 3 and a.world_size() == 1 and a.world_rank() == 0 and a.is_mixed_precision()
    assert a.to_fp32(a.to_fp16(torch.ones(3))).dtype == torch.float32
    a.unflatten_params()
    text = a.print_memory_profile()
    assert "optimizer state" in text and "unsharded total" in capsys.readouterr().out
    blk = FSDPBlock(a, 0)
    assert blk.memory_usage() > 0 and len(blk.sync_gradients()) == len(blk.weights)
    # the block alone: forward keeps what backward needs; backward returns the input gradient and refreshes the shards
    h = torch.randn(32, 32)
    eng = a.engine
    ref_out, ref_ctx = eng._block_fwd(0, h, 2, 16)
    out = blk.forward(h, 2, 16)
    assert torch.equal(out, ref_out)
    dy = torch.randn_like(out)
    eng.gshard.zero_()
    dh = blk.backward(dy)
    hp = h.clone().requires_grad_(True)
    assert dh.shape == h.shape and any(float(g.abs().sum()) > 0 for g in blk.shard_gradients())
    eps = 1e-3
    d = torch.randn_like(h)
    num = float(((eng._block_fwd(0, h + eps * d, 2, 16)[0] - eng._block_fwd(0, h - eps * d, 2, 16)[0]) * dy).sum()) / (2 * eps)
    assert num == pytest.approx(float((dh * d).sum()), rel=2e-2, abs=1e-3)
    with pytest.raises(RuntimeError):
        blk.backward(dy)
    # explicit activation checkpointing: the recomputed output carries gradients back to the saved input
    lin = torch.nn.Linear(8, 8)
    ac = ActivationCheckpointing()
    x = torch.randn(4, 8)
    ac.save_input(3, x)
    assert ac.saved_memory() == x.numel() * 4
    y = ac.recompute(lin, 3)
    y.sum().backward()
    assert torch.allclose(y, lin(x)) and lin.weight.grad is not None
    ac.clear()
    assert ac.saved_memory() == 0
    # per-shard optimizer: both forms descend on a quadratic; the mixed form keeps the master exact and the shard rounded
    opt = ZeROOptimizer(lr=5e-2, weight_decay=0.0)
    w = torch.randn(16, 8, generator=torch.Generator().manual_seed(2))
    target = torch.zeros_like(w)
    w_lp, master = w.to(torch.bfloat16), w.clone()
    start = float(w.pow(2).sum())
    for t in range(1, 60):
        opt.step(w, 2 * (w - target), t)
        opt.step_mixed(w_lp, master, 2 * (master - target), t)
    assert float(w.pow(2).sum()) < 0.2 * start and float(master.pow(2).sum()) < 0.2 * start
    assert torch.equal(w_lp, master.to(torch.bfloat16))
    opt.set_param_count(128)
    assert opt.param_count() == 128


def test_zero_optimizer_stage3_verbs_single_process():
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.parallel.fsdp import ZeroOptimizer
    m = DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=1, num_heads=4, ffn_hidden_size=64, max_seq_len=16),
                   device="cpu", dtype=torch.float32, seed=0)
    z = ZeroOptimizer(m, 0, 1, lr=1e-2, stage=2)
    z.set_grad_clip_norm(0.5)
    ids = torch.randint(0, 64, (2, 16))
    m.forward_backward(ids, torch.roll(ids, -1, 1))
    n = z.clip_grad_norm()
    assert n > 0.5 and float(m.flat.grads.norm()) == pytest.approx(0.5, rel=1e-4)
    assert z.reduce_scatter_grads().numel() == z.num_owned() and z.all_gather_params() is m.flat.params
    assert z.state_bytes_owned() == z.state_bytes_full() and z.world_size() == 1


def test_activation_checkpoint_regions_measure_and_place():
    from transformers_fusion_b200.parallel.fsdp import ActivationCheckpoint, MemoryBudget
    ac = ActivationCheckpoint()
    blocks = [torch.nn.Sequential(torch.nn.Linear(32, w), torch.nn.GELU(), torch.nn.Linear(w, 32)) for w in (64, 256, 128)]
    x = torch.randn(16, 32, requires_grad=True)
    h = x
    for i, blk in enumerate(blocks):
        with ac.region(f"block{i}") as info:
            h = blk(h)
        assert not ac.in_checkpoint_region()
    sizes = [r.forward_activations_bytes for r in ac.regions()]
    # each block saves its input [16, 32], the pre-activation and the activation [16, w]: 4 bytes each
    assert sizes == [16 * (32 + 2 * w) * 4 for w in (64, 256, 128)]
    assert ac.auto_place_checkpoints() == []                           # no budget: nothing to do
    total = sum(sizes)
    ac.set_budget(MemoryBudget(total_bytes=total + 1000, param_bytes=600, grad_bytes=300, opt_state_bytes=100 + sizes[1] - 10))
    assert ac.auto_place_checkpoints() == ["block1"]                   # dropping the largest region is enough
    assert ac.estimated_savings_all() == sizes[1] and ac.budget.activation_bytes == total - sizes[1]
    ac.begin_region("declared", "FULL", activation_bytes=4096, recompute_flops=8192)
    assert ac.in_checkpoint_region()
    ac.end_region()
    assert ac.total_activations_saved() == sizes[1] + 4096 and ac.compute_overhead() == pytest.approx((1 + 8192) / (sizes[1] + 4096))
    assert ActivationCheckpoint.estimate_layer_activations(2, 128, 64, 256) == 2 * 128 * (512 + 768) * 2
    ac.reset()
    assert ac.regions() == [] and ac.compute_overhead() == 0.0


def test_offload_engine_and_manager_reference_verbs():
    from transformers_fusion_b200.parallel.fsdp import CPUOffloadEngine, GradientCheckpointManager, ZeROOffloadManager
    eng = CPUOffloadEngine(pool_bytes=1 << 20, device="cpu")
    a, b = torch.arange(8.0), torch.arange(4.0) + 10
    eng.offload_params([a, b])
    keep = a.clone()
    a.zero_()
    eng.prefetch_params([0])
    assert torch.equal(a, keep) and eng.bytes_offloaded() == 48 and eng.bytes_prefetched() == 32
    b.zero_()
    eng.prefetch_all()
    assert b.tolist() == [10.0, 11.0, 12.0, 13.0]
    dst = torch.zeros(4)
    eng.async_transfer(dst, torch.ones(4))
    eng.synchronize()
    assert dst.sum() == 4 and not eng.is_busy() and eng.pending_transfers() == 0
    comp, tr = torch.zeros(2), torch.zeros(2)
    comp, tr = eng.double_buffer_transfer(comp, tr, torch.tensor([5.0, 6.0]))
    assert comp.tolist() == [5.0, 6.0] and eng.pin_memory(a) is a and CPUOffloadEngine.unpin_memory(a) is a
    eng.reset_stats(), eng.clear()
    assert eng.bytes_offloaded() == 0 and eng.used == 0

    class Opt:
        m, v = torch.ones(6), torch.full((6,), 2.0)
    mgr = ZeROOffloadManager(Opt(), CPUOffloadEngine(1 << 20, "cpu"))
    assert mgr.bytes_on_device() == 48 and mgr.offload_ratio() == 0.0
    m, v = torch.ones(3), torch.full((3,), 4.0)
    mgr.offload_optimizer_state(m, v, 7)
    m.zero_(), v.zero_()
    assert mgr.bytes_offloaded() == 24 and 0 < mgr.offload_ratio() < 1
    mgr.reload_optimizer_state(m, v, 7)
    assert m.tolist() == [1.0] * 3 and v.tolist() == [4.0] * 3
    g = torch.arange(10.0)
    parts = [ZeROOffloadManager.shard_gradient(g, r, 4) for r in range(4)]
    assert [p.tolist() for p in parts] == [[0, 1, 2], [3, 4, 5], [6, 7, 8], [9, 0, 0]]
    full = sum(ZeROOffloadManager.unshard_gradient(p, r, 4, 10) for r, p in enumerate(parts))
    assert torch.equal(full, g)
    mgr.reset_stats()
    G = GradientCheckpointManager
    G.reset_stats()
    G.begin_checkpoint(1000)
    assert G.in_checkpoint()
    G.end_checkpoint()
    G.begin_checkpoint(500), G.end_checkpoint(recomputed=False)
    assert not G.in_checkpoint() and G.activations_saved() == 2 and G.activations_recomputed() == 1
    assert G.memory_saved_bytes() == 1500 and G.compute_overhead() == 0.5
    G.reset_stats()
    assert G.activations_saved() == 0


def test_zero_optimizer_parameter_counts_and_checkpoint_budget_access():
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.parallel.fsdp import ActivationCheckpoint, ZeroOptimizer
    m = DenseModel(TransformerConfig(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, ffn_hidden_size=64, max_seq_len=16), device="cpu",
                   dtype=torch.float32, seed=0)
    z = ZeroOptimizer(m, 0, 1, stage=1)
    assert z.total_params() == len(m.flat.params_list) == z.owned_params() and z.register_model_params() == z.total_params()
    ac = ActivationCheckpoint()
    ac.mutable_budget().total_bytes = 12345
    assert ac.budget.total_bytes == 12345
