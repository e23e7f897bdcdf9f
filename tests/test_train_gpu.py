"""End-to-end training step on the GPU: bf16 kernels against the CPU fp32 statement of the same
model, loss decrease, CUDA-graph replay equivalence."""
import pytest
import torch

from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.ops import _lib
from transformers_fusion_b200.trainer.engine import TrainEngine

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    base = dict(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=512,
                max_seq_len=256, init_std=0.05)
    base.update(kw)
    return TransformerConfig(**base)


@pytest.mark.parametrize("kw", [dict(), dict(tie_embeddings=True, use_parallel_residual=True),
                                dict(activation="gelu", norm_type="layernorm", position_type="learned",
                                     attention_bias=True, tie_embeddings=True)])
def test_grads_match_cpu_fp32(kw):
    cfg = _cfg(**kw)
    ref = DenseModel(cfg, dtype=torch.float32, seed=5)
    ref.flatten()
    gpu = DenseModel(cfg, device="cuda", dtype=torch.bfloat16, seed=5)
    gpu.flatten()
    ref.flat.params.copy_(gpu.flat.params.float().cpu())  # identical (bf16-rounded) weights
    ids = torch.randint(0, cfg.vocab_size, (2, 256))
    labels = torch.roll(ids, -1, 1)
    l_ref = ref.forward_backward(ids, labels)
    l_gpu = gpu.forward_backward(ids.cuda(), labels.cuda())
    torch.cuda.synchronize()
    _lib.check_status()
    assert abs(l_ref.item() - l_gpu.item()) < 3e-2
    g_ref, g_gpu = ref.flat.grads, gpu.flat.grads.cpu()
    cos = torch.nn.functional.cosine_similarity(g_ref, g_gpu, dim=0).item()
    assert cos > 0.99, cos
    rel = (g_ref - g_gpu).norm().item() / g_ref.norm().item()
    assert rel < 0.1, rel


def test_loss_decreases_and_graph_matches_eager():
    cfg = _cfg(tie_embeddings=True)
    ids = torch.randint(0, cfg.vocab_size, (4, 256), device="cuda")
    labels = torch.roll(ids, -1, 1)
    losses = {}
    for graph in (False, True):
        model = DenseModel(cfg, device="cuda", dtype=torch.bfloat16, seed=7)
        eng = TrainEngine(model, lr=1e-3, cuda_graph=graph)
        ls = [float(eng.step(ids, labels).item()) for _ in range(8)]
        losses[graph] = ls
        assert ls[-1] < ls[0] - 0.2, ls
    torch.cuda.synchronize()
    _lib.check_status()
    for a, b in zip(losses[False], losses[True]):
        assert abs(a - b) < 5e-2, (losses[False], losses[True])


def test_activation_checkpointing_same_grads():
    cfg = _cfg()
    ids = torch.randint(0, cfg.vocab_size, (2, 256), device="cuda")
    labels = torch.roll(ids, -1, 1)
    gs = []
    for ck in (False, True):
        m = DenseModel(cfg, device="cuda", dtype=torch.bfloat16, seed=9)
        m.flatten()
        m.activation_checkpointing = ck
        m.forward_backward(ids, labels)
        gs.append(m.flat.grads.clone())
    torch.cuda.synchronize()
    rel = (gs[0] - gs[1]).norm().item() / gs[0].norm().item()
    assert rel < 2e-2, rel   # split-K atomics reorder fp32 sums; nothing else differs


@pytest.mark.gpu
def test_fused_adafactor_matches_pytorch_statement():
    """Multi-tensor Adafactor kernels (csrc/kernels/adafactor.cu) against the per-tensor PyTorch statement in fp32."""
    import torch
    from transformers_fusion_b200.models.config import TransformerConfig
    from transformers_fusion_b200.models.dense import DenseModel
    from transformers_fusion_b200.trainer.optimizers import Adafactor
    cfg = TransformerConfig(vocab_size=256, hidden_size=128, num_layers=2, num_heads=2, ffn_hidden_size=256, max_seq_len=64)
    for beta1 in (0.0, 0.9):
        a = DenseModel(cfg, device="cuda", dtype=torch.bfloat16, seed=1)
        b = DenseModel(cfg, device="cuda", dtype=torch.bfloat16, seed=1)
        fa, fb = a.flatten(), b.flatten()
        oa = Adafactor(fa, lr=1e-2, weight_decay=0.01, max_grad_norm=1.0, beta1=beta1)
        ob = Adafactor(fb, lr=1e-2, weight_decay=0.01, max_grad_norm=1.0, beta1=beta1)
        ob._fused_tables = lambda: None                    # force the PyTorch statement
        g = torch.Generator(device="cuda").manual_seed(0)
        for step in range(3):
            gr = torch.randn(fa.numel, device="cuda", generator=g) * 0.1
            fa.grads.copy_(gr)
            fb.grads.copy_(gr)
            oa.step()
            ob.step()
            err = (oa.master - ob.master).abs().max().item()
            assert err < 2e-5, (beta1, step, err)
            assert float(fa.grads.abs().max()) == 0.0
        assert torch.equal(fa.params, oa.master.to(torch.bfloat16))
