"""Hand-written forward/backward of the dense model against torch autograd on an independent
PyTorch implementation (CPU, fp32), including GQA, parallel residual, checkpointing and the
GPT-2-shaped variant."""
import math

import pytest
import torch
import torch.nn.functional as TF

from transformers_fusion_b200.models.config import TransformerConfig
from transformers_fusion_b200.models.dense import DenseModel
from transformers_fusion_b200.ops import functional as F


def ref_forward(model, ids):
    cfg = model.cfg
    B, S = ids.shape
    Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    p = {n: t.detach().clone().double().requires_grad_(True) for n, t in model.named_tensors()}
    x = p["tok_embeddings.weight"][ids]
    if cfg.position_type == "learned":
        x = x + p["pos_embeddings.weight"][:S]
    cos, sin = F.rope_tables(D, cfg.max_seq_len, cfg.rope_theta)
    cos, sin = cos[:S].double(), sin[:S].double()

    def norm(h, name):
        if cfg.norm_type == "layernorm":
            return TF.layer_norm(h, (h.shape[-1],), p[name + ".weight"], p[name + ".bias"], cfg.norm_eps)
        return h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * p[name + ".weight"]

    def lin(h, name):
        y = h @ p[name + ".weight"].t()
        if name + ".bias" in p:
            y = y + p[name + ".bias"]
        return y

    def rope(t):
        half = D // 2
        t1, t2 = t[..., :half], t[..., half:]
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.cat([t1 * c - t2 * s, t2 * c + t1 * s], -1)

    for i in range(cfg.num_layers):
        pre = f"layers.{i}."
        a = norm(x, pre + "attention_norm")
        q = lin(a, pre + "attention.q_proj").view(B, S, Hq, D)
        k = lin(a, pre + "attention.k_proj").view(B, S, Hkv, D)
        v = lin(a, pre + "attention.v_proj").view(B, S, Hkv, D)
        if cfg.position_type == "rope":
            q, k = rope(q), rope(k)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        k = k.repeat_interleave(Hq // Hkv, 1)
        v = v.repeat_interleave(Hq // Hkv, 1)
        s = q @ k.transpose(-1, -2) / math.sqrt(D)
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
        o = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, S, Hq * D)
        attn = lin(o, pre + "attention.o_proj")
        if cfg.use_parallel_residual:
            f = norm(x, pre + "ffn_norm")
        else:
            x = x + attn
            f = norm(x, pre + "ffn_norm")
        if cfg.gated:
            g = lin(f, pre + "ffn.gate_proj")
            u = lin(f, pre + "ffn.up_proj")
            act = (TF.silu(g) if cfg.activation == "swiglu" else TF.gelu(g, approximate="tanh")) * u
        else:
            u = lin(f, pre + "ffn.up_proj")
            act = {"gelu": lambda t: TF.gelu(t, approximate="tanh"), "relu": torch.relu, "silu": TF.silu}[cfg.activation](u)
        ffn = lin(act, pre + "ffn.down_proj")
        x = x + ffn + (attn if cfg.use_parallel_residual else 0)
    x = norm(x, "norm")
    head = p["tok_embeddings.weight"] if cfg.tie_embeddings else p["lm_head.weight"]
    return x @ head.t(), p


CASES = {
    "llama_gqa": dict(vocab_size=97, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, ffn_hidden_size=96,
                      max_seq_len=32),
    "tied_parallel": dict(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, ffn_hidden_size=48, max_seq_len=16,
                          tie_embeddings=True, use_parallel_residual=True, activation="geglu"),
    "gpt2ish": dict(vocab_size=80, hidden_size=32, num_layers=2, num_heads=2, ffn_hidden_size=64, max_seq_len=16,
                    activation="gelu", norm_type="layernorm", position_type="learned", attention_bias=True,
                    tie_embeddings=True),
}


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("ckpt", [False, True])
def test_forward_backward_matches_autograd(name, ckpt):
    cfg = TransformerConfig(**CASES[name], init_std=0.2)
    model = DenseModel(cfg, dtype=torch.float32, seed=1)
    with torch.no_grad():
        for n, prm in model.named_parameters():
            if prm.dim() == 1:
                prm.add_(0.1 * torch.randn_like(prm))
    model.flatten()
    model.activation_checkpointing = ckpt
    B, S = 2, 12
    ids = torch.randint(0, cfg.vocab_size, (B, S))
    labels = torch.randint(0, cfg.vocab_size, (B, S))
    labels[0, 3] = -100
    loss = model.forward_backward(ids, labels)
    logits, p = ref_forward(model, ids)
    ref_loss = TF.cross_entropy(logits.view(B * S, -1), labels.view(-1), ignore_index=-100)
    ref_loss.backward()
    assert abs(loss.item() - ref_loss.item()) < 1e-4
    grads = dict(zip([n for n, _ in model.named_tensors()], [None] * 1000))
    # map views back to main_grad slices
    D = cfg.head_dim
    nq, nkv, Fh = cfg.num_heads * D, cfg.num_kv_heads * D, cfg.ffn_hidden_size
    for n, t in model.named_tensors():
        g = p[n].grad
        assert g is not None, n
        # locate our gradient: walk the flat buffer by data_ptr offset
        off = (t.data_ptr() - model.flat.params.data_ptr()) // t.element_size()
        ours = model.flat.grads[off: off + t.numel()].view(t.shape)
        assert torch.allclose(ours.double(), g, atol=2e-4, rtol=2e-3), (n, (ours.double() - g).abs().max().item())


def test_autograd_path_matches_fused_path():
    cfg = TransformerConfig(**CASES["llama_gqa"], init_std=0.2)
    model = DenseModel(cfg, dtype=torch.float32, seed=3)
    model.flatten()
    ids = torch.randint(0, cfg.vocab_size, (2, 8))
    labels = torch.randint(0, cfg.vocab_size, (2, 8))
    loss = model.forward_backward(ids, labels)
    g1 = model.flat.grads.clone()
    model.flat.zero_grad()
    logits = model(ids)
    l2 = TF.cross_entropy(logits.float().view(16, -1), labels.view(-1))
    l2.backward()
    assert abs(l2.item() - loss.item()) < 1e-4
    assert torch.allclose(model.flat.grads, g1, atol=1e-4, rtol=1e-3)


def test_config_binary_roundtrip():
    cfg = TransformerConfig(vocab_size=32000, hidden_size=512, num_layers=8, num_heads=8, ffn_hidden_size=1408,
                            num_kv_heads=4, rope_scaling_mode="yarn", rope_scaling_factor=4.0, mtp_num_heads=2,
                            mtp_loss_weight=0.3, use_parallel_residual=True)
    raw = cfg.to_bytes()
    assert len(raw) == 128
    back = TransformerConfig.from_bytes(raw)
    for k in ("vocab_size", "hidden_size", "num_layers", "num_heads", "head_dim", "ffn_hidden_size", "max_seq_len",
              "activation", "num_kv_heads", "use_parallel_residual", "mtp_num_heads", "rope_scaling_mode"):
        assert getattr(back, k) == getattr(cfg, k), k
    assert abs(back.rope_scaling_factor - 4.0) < 1e-6 and abs(back.mtp_loss_weight - 0.3) < 1e-6


def test_multi_token_prediction_heads_train_and_files_roundtrip(tmp_path):
    """The fused step with extra prediction heads equals the autograd statement (main CE + weight x mean of the heads' CE
    on labels shifted further left), and save / save_quantized / load keep the heads."""
    from transformers_fusion_b200.models.dense import _LinearFn
    cfg = TransformerConfig(**CASES["llama_gqa"], init_std=0.2, mtp_num_heads=2, mtp_loss_weight=0.3)
    model = DenseModel(cfg, dtype=torch.float32, seed=4)
    model.flatten()
    B, S = 2, 8
    ids = torch.randint(0, cfg.vocab_size, (B, S))
    labels = torch.randint(0, cfg.vocab_size, (B, S))
    labels[1, 2] = -100
    loss = model.forward_backward(ids, labels)
    g1 = model.flat.grads.clone()
    assert all(h.main_grad.abs().sum() > 0 for h in model.mtp_heads)
    model.flat.zero_grad()
    f = model.hidden_states(ids)
    want = TF.cross_entropy(_LinearFn.apply(f, model.lm_head).float(), labels.view(-1), ignore_index=-100)
    shifted = model.mtp_shifted_labels(labels)
    assert shifted[0].view(B, S)[0, :-1].tolist() == labels[0, 1:].tolist() and shifted[1].view(B, S)[0, -2:].tolist() == [-100, -100]
    for w, lab in zip(model.mtp_heads, shifted):
        want = want + 0.3 / 2 * TF.cross_entropy(_LinearFn.apply(f, w).float(), lab, ignore_index=-100)
    want.backward()
    assert abs(want.item() - loss.item()) < 1e-4
    assert torch.allclose(model.flat.grads, g1, atol=1e-4, rtol=1e-3)
    # without the weight the heads are left alone
    model.flat.zero_grad()
    model.mtp_loss_weight = 0.0
    model.forward_backward(ids, labels)
    assert all(float(h.main_grad.abs().sum()) == 0 for h in model.mtp_heads)
    # files
    path = model.save(str(tmp_path / "m.quant"))
    back = DenseModel.load(path)
    assert len(back.mtp_heads) == 2 and torch.equal(back.mtp_heads[1].data, model.mtp_heads[1].data)
    with torch.no_grad():
        a, b = model.mtp_forward(ids), back.mtp_forward(ids)
    assert len(a) == 2 and a[0].shape == (B, S, cfg.vocab_size) and torch.allclose(a[1], b[1], atol=1e-6)
    q = DenseModel.load(model.save_quantized(str(tmp_path / "m8.quant"), "Q_8"))
    with torch.no_grad():
        full = model(ids)
        err = (q(ids) - full).abs().max()
    assert 0 < float(err) < 0.05 * float(full.abs().max())


def test_rotary_embedding_object_rotates_and_inverts():
    from transformers_fusion_b200.models.dense import RotaryEmbedding
    cfg = TransformerConfig(**CASES["llama_gqa"])
    r = RotaryEmbedding.from_config(cfg)
    x = torch.randn(2 * 12, cfg.num_heads * cfg.head_dim)
    y = r(x, cfg.num_heads, 12)
    assert (y - x).abs().max() > 0 and torch.allclose(y.view(24, cfg.num_heads, -1).norm(dim=-1), x.view(24, cfg.num_heads, -1).norm(dim=-1), atol=1e-5)
    assert torch.allclose(r.apply_(y.clone(), cfg.num_heads, 12, inverse=True), x, atol=1e-5)
    lin = RotaryEmbedding(cfg.head_dim, 32, scaling_mode="linear", scaling_factor=2.0)
    assert torch.allclose(lin.cos[2], r.cos[1], atol=1e-6)            # positions are divided by the factor
