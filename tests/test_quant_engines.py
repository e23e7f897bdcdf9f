import math
import pytest
import torch

from transformers_fusion_b200.quant import engines as E


def test_codebook_train_and_serialize():
    torch.manual_seed(0)
    x = torch.randn(50000) * 0.3
    errs = []
    for bits in (3, 4, 6, 8):
        cb = E.Codebook(bits)
        e0 = E.quant_error(x, cb.dequantize(cb.quantize(x)))
        cb.train(x)
        e1 = E.quant_error(x, cb.dequantize(cb.quantize(x)))
        assert e1 < e0 and cb.centroids.numel() == 1 << bits and bool((cb.centroids[1:] >= cb.centroids[:-1]).all())
        errs.append(e1)
        cb2 = E.Codebook.deserialize(cb.serialize())
        assert len(cb.serialize()) == cb.serialized_size()
        assert torch.allclose(cb2.centroids, cb.centroids, atol=2e-3 if bits < 8 else 0)
    assert errs == sorted(errs, reverse=True)          # more bits, less error
    cb = E.CodebookQ4().train(x)
    before = cb.centroids.clone()
    cb.ema_update(x + 0.5, cb.quantize(x), 0.5)
    assert float((cb.centroids - before).mean()) == pytest.approx(0.25, abs=0.02)


def test_vector_quantizer():
    torch.manual_seed(1)
    centers = torch.randn(8, 4) * 3
    x = centers[torch.randint(0, 8, (2000,))] + 0.05 * torch.randn(2000, 4)
    vq = E.VectorQuantizer(8, 4).train(x)
    q, idx, loss = vq.forward(x.clone().requires_grad_())
    assert float(loss.detach()) < 0.1 and idx.shape == (2000,) and q.requires_grad
    q.sum().backward()                                   # straight-through


def test_engines_roundtrip_and_snr():
    torch.manual_seed(2)
    w = torch.randn(1000, 70) * 0.05
    snr = {}
    for name, eng in (("q8", E.Q8Engine()), ("q4", E.Q4Engine()), ("q2", E.Q2Engine())):
        eng.train_codebook_per_block(w)
        snr[name] = E.quant_snr(w, eng.roundtrip(w))
    assert snr["q8"] > 30 and snr["q8"] > snr["q4"] > snr["q2"] > 3
    st = E.Q4Engine(stochastic=True).train_codebook_per_block(w)
    avg = torch.stack([st.roundtrip(w[:64]) for _ in range(200)]).mean(0)
    det = E.Q4Engine().train_codebook_per_block(w).roundtrip(w[:64])
    assert E.quant_error(w[:64], avg) < 0.5 * E.quant_error(w[:64], det)       # stochastic rounding is unbiased
    t = E.QuantEngine()
    p, s = t.quantize(w)
    d = t.dequantize(p, s, w.numel()).view(w.shape)
    assert p.numel() == ((w.numel() + 127) // 128 * 128) // 4 and set(torch.unique(torch.round(d.reshape(-1)[:128] / s[0])).tolist()) <= {-1.0, 0.0, 1.0}
    a = torch.randn(3, 70)
    assert torch.allclose(t.quant_gemm(a, p, s, 3, 1000, 70), a @ d.t(), atol=1e-5)
    q, sc = t.quantize_per_channel(w, 0)
    assert q.shape == w.shape and sc.shape == (1000,) and t.dequantize_per_channel(q, sc, 0).shape == w.shape
    b, sc1 = E.Q1Engine().quantize(w)
    d1 = E.Q1Engine().dequantize(b, sc1, w.numel())
    assert torch.equal(torch.sign(d1), torch.where(w.view(-1) >= 0, 1.0, -1.0)) and E.quant_snr(w, d1.view(w.shape)) > 2
    assert E.Q32Engine().dequantize(E.Q32Engine().quantize(w)).equal(w)
    assert E.quant_snr(w, E.Q16Engine().dequantize(E.Q16Engine().quantize(w))) > 60


def test_fp8_and_quant8():
    torch.manual_seed(3)
    x = torch.randn(64, 32) * 10
    for kind, tol in (("e4m3", 0.07), ("e5m2", 0.13)):
        q, s = E.fp8_quantize(x, kind)
        assert float((E.fp8_dequantize(q, s) - x).abs().max() / x.abs().max()) < tol
    q, s = E.fp8_quantize(x, "e4m3", per_channel_dim=0)
    assert s.shape == (64, 1) and float(q.float().abs().max()) <= 448
    big, _ = E.fp8_quantize(torch.tensor([1e9, -1e9, 1.0]), "e4m3")
    assert torch.isfinite(big.float()).all()                # e4m3 has no infinities: saturates at 448
    a, b = torch.randn(8, 32), torch.randn(5, 32)
    assert float((E.fp8_quant_gemm(a, b) - a @ b.t()).abs().max()) < 0.8
    for sym in (False, True):
        q, s, zp = E.quant8_quantize_tensor(x, sym)
        assert float((E.quant8_dequantize_tensor(q, s, zp) - x).abs().max()) <= s * 0.51 + 1e-6


def test_ternary_lut_streams():
    """TL1 / TL2 row streams: byte layout, round trip at ragged K, the lookup-table product's integer arithmetic (written
    out here as the reference's scalar loops), and the transcode to the packed device format."""
    torch.manual_seed(3)
    for kind, K in ((1, 10), (1, 13), (2, 24), (2, 29)):
        tl = E.TernaryLUT(kind)
        t = torch.randint(-1, 2, (5, K))
        packed = tl.pack(t)
        assert packed.shape == (5, (K + 3) // 4 if kind == 1 else (K + 11) // 12 * 3) and packed.dtype == torch.uint8
        assert torch.equal(tl.unpack(packed, K).long(), t)
        # weight i of a row sits in bits 2 * (i % 4) of byte i // 4, with 00 = -1, 01 = 0, 10 = +1
        for i in range(K):
            assert int((packed[2, i // 4] >> (2 * (i % 4))) & 3) == int(t[2, i]) + 1
        a = torch.randn(3, K) * 2
        got = tl.gemm(packed, a, K)
        want = torch.zeros(5, 3)
        for n in range(3):
            sc = 127.0 / max(float(a[n].abs().max()), 1e-10)
            ai = torch.round(a[n] * sc).long()
            for m in range(5):
                if kind == 1:
                    tot = 0
                    for i in range(0, K - 1, 2):
                        tot += max(-128, min(127, int(ai[i]) * int(t[m, i]) + int(ai[i + 1]) * int(t[m, i + 1])))
                    if K % 2:
                        tot += int(ai[K - 1]) * int(t[m, K - 1])
                else:
                    tot = int((ai * t[m]).sum())
                want[m, n] = tot / sc
        assert torch.allclose(got, want, atol=1e-5), (kind, K)
        if kind == 2:          # no saturation: off the exact product only by the int8 rounding of the activations
            assert (got - t.float() @ a.t()).abs().max() <= 0.5 * K * float(a.abs().max()) / 127 + 1e-5
    # transcode for the fused-dequant GEMM: ternary values x per-row scale survive exactly
    tl = E.TernaryLUT(1)
    t = torch.randint(-1, 2, (128, 64))
    scale = torch.rand(128) + 0.5
    pw = tl.to_packed_weight(tl.pack(t), 64, scale)
    from transformers_fusion_b200.quant import wq
    assert torch.allclose(wq.dequant(pw)[:128, :64], t.float() * scale[:, None], rtol=1e-2, atol=1e-3)


def test_engine_verbs_shared_by_all_widths():
    import torch
    from transformers_fusion_b200.quant import engines as E
    g = torch.Generator().manual_seed(0)
    w = torch.randn(16, 64, generator=g)
    a = torch.randn(4, 64, generator=g)
    for cls, tol in ((E.Q8Engine, 0.05), (E.Q4Engine, 0.35), (E.Q2Engine, 0.9)):
        e = cls(block_size=64).train_codebook_per_block(w)
        assert e.codebook().numel() == 2 ** e.bits
        idx, sc = e.quantize_per_block(w, 32)
        assert sc.numel() == 32 and idx.numel() == w.numel()
        back = e.dequantize_per_block(idx, sc, w.numel(), 32).view_as(w)
        assert e.quant_error(w, back) < tol and e.quant_snr(w, back) > 0
        qt = e.quantize_tensor(w)
        assert torch.allclose(e.quant_gemm(a, qt, 4, 16, 64), a @ e.dequant_tensor(qt).view(16, 64).t(), atol=1e-5)
        i2, s2 = e.quantize(w)
        assert torch.allclose(e.quant_gemm(a, i2, 4, 16, 64, scales=s2), a @ e.dequantize(i2, s2, w.numel()).view(16, 64).t(), atol=1e-5)
        qc, scs = e.quantize_per_channel(w, 0)
        assert qc.shape == w.shape and scs.shape == (16,)
        assert e.quant_error(w, e.dequantize_per_channel(qc, scs, 0)) < tol
        qc1, scs1 = e.quantize_per_channel(w, 1)
        assert scs1.shape == (64,) and e.dequantize_per_channel(qc1, scs1, 1).shape == w.shape
        e.enable_stochastic_rounding(True, 0.5)
        assert e.stochastic and e.stoch_temperature == 0.5
    for cls, exact in ((E.Q32Engine, True), (E.Q16Engine, False)):
        e = cls()
        q = e.quantize_batch(w)
        assert torch.equal(e.dequantize_batch(q), w) == exact and e.quant_error(w, e.dequantize(q)) < 1e-3
        assert torch.allclose(e.quant_gemm(a, q, 4, 16, 64), a @ w.t(), atol=1e-2)
        qc, sc = e.quantize_per_channel(w, 0)
        assert torch.allclose(e.dequantize_per_channel(qc, sc, 0), w, atol=1e-3)
    q1 = E.Q1Engine()
    packed = q1.quantize_batch(w)
    assert torch.equal(q1.dequantize_batch(packed)[: w.numel()].sign(), torch.where(w.reshape(-1) >= 0, 1.0, -1.0))
    qc, sc = q1.quantize_per_channel(w, 0)
    assert torch.equal(q1.dequantize_per_channel(qc, sc, 0).sign(), torch.where(w >= 0, 1.0, -1.0))
    # fp8 by name: exact values of the encodings
    assert E.fp8_e4m3_dequantize(E.fp8_e4m3_quantize(1.0)) == 1.0 and E.fp8_e4m3_dequantize(E.fp8_e4m3_quantize(1e6)) == 448.0
    assert E.fp8_e5m2_dequantize(E.fp8_e5m2_quantize(-1e9)) == -57344.0 and E.fp8_e5m2_quantize(0.0) == 0
    bits = E.fp8_e4m3_quantize_tensor(w)
    assert bits.dtype == torch.uint8 and E.fp8_e4m3_quant_error(w, E.fp8_e4m3_dequant_tensor(bits)) < 0.08
    assert torch.allclose(E.fp8_e4m3_quant_gemm(a, bits, 4, 16, 64), a @ E.fp8_e4m3_dequant_tensor(bits).t(), atol=1e-5)
    qch, sch = E.fp8_e5m2_quantize_per_channel(w, 0)
    assert qch.dtype == torch.uint8 and E.fp8_e5m2_quant_snr(w, E.fp8_e5m2_dequantize_per_channel(qch, sch, 0)) > 15
    assert E.compute_quant_mse(w, w) == 0.0 and E.compute_quant_error(w, w) == 0.0


def test_vector_quantizer_online_updates_and_usage_statistics():
    torch.manual_seed(0)
    centres = torch.tensor([[4.0, 4.0], [-4.0, 4.0], [4.0, -4.0], [-4.0, -4.0]])
    x = (centres[torch.randint(0, 4, (2, 256))] + 0.1 * torch.randn(2, 256, 2))
    vq = E.VectorQuantizer(E.VQConfig(codebook_size=4, embedding_dim=2, ema_decay=0.5, codebook_init_std=4.0), seed=1)
    assert vq.config().codebook_size == 4 and vq.codebook().shape == (4, 2) and vq.perplexity() == 0.0
    first = vq.quantize(x)
    assert first.quantized.shape == x.shape and first.indices.shape == (2, 256) and first.codebook_loss == 0.0
    for _ in range(30):
        r = vq.quantize(x)
        vq.update_ema(x, r.indices)
    last = vq.quantize(x)
    assert last.commitment_loss < 0.6 * first.commitment_loss         # k-means can still leave one code serving two clusters
    used = int((vq._hits > 0).sum())
    assert vq.usage_rate() == used / 4 and 1.0 <= vq.perplexity() <= used + 1e-4
    g = torch.randn(2, 256, 2)
    assert vq.backward(g) is g
    # the gradient form: a step against the gradient of ||q - x||^2 / 2 moves every used code toward its members
    vg = E.VectorQuantizer(E.VQConfig(codebook_size=4, embedding_dim=2, use_ema=False, codebook_init_std=4.0), seed=1)
    r0 = vg.quantize(x)
    assert r0.codebook_loss == r0.commitment_loss
    for _ in range(50):
        r = vg.quantize(x)
        n = torch.bincount(r.indices.reshape(-1), minlength=4).clamp(min=1)[r.indices.reshape(-1)]
        vg.update_codebook_grad(((r.quantized - x).reshape(-1, 2) / n[:, None]), r.indices, lr=0.5)
    assert vg.quantize(x).commitment_loss < r0.commitment_loss


def test_min_max_observer_interface():
    from transformers_fusion_b200.quant import qat as Q
    o = Q.MinMaxObserver()
    assert not o.has_data() and o.calc_qparams(8, True).scale == 1.0 and o.type() == "MinMax" and o.min_val() == 0.0
    o.observe(torch.tensor([-1.0, 0.5])), o.observe(torch.tensor([0.25, 3.0]))
    assert o.min_val() == -1.0 and o.max_val() == 3.0
    sp = o.calc_qparams(8, True)
    assert sp.zero_point == 0 and sp.qmax == 127 and sp.scale == pytest.approx(3.0 / 127)
    ap = o.calc_qparams(8, False)
    x = torch.tensor([-1.0, 0.0, 1.7, 3.0])
    assert ap.qmin == 0 and ap.qmax == 255 and float(ap.dequantize(ap.quantize(torch.zeros(1)))) == 0.0
    assert (ap.dequantize(ap.quantize(x)) - x).abs().max() <= ap.scale / 2 + 1e-6
    o.reset()
    assert not o.has_data()
    m = Q.MovingAverageObserver(0.5)
    m.observe(torch.tensor([0.0, 2.0])), m.observe(torch.tensor([0.0, 4.0]))
    assert m.max_val() == 3.0 and m.type() == "MovingAverage"
    m.reset(), m.observe(torch.tensor([0.0, 8.0]))
    assert m.max_val() == 8.0


def test_qat_objects_lsq_quantizer_kl_observer_and_context():
    from transformers_fusion_b200.quant import qat as Q
    assert Q.get_qrange(8) == (-128, 127) and Q.get_qrange(8, True, True) == (-127, 127) and Q.get_qrange(4, False) == (0, 15)
    assert Q.get_qrange(Q.QATConfig(bits=4, narrow_range=True)) == (-7, 7)
    x = torch.randn(4096)
    xg = x.clone().requires_grad_(True)
    y = Q.fake_quantize_per_tensor(xg, 0.05, 8)
    y.sum().backward()
    assert torch.equal(xg.grad, torch.ones_like(x)) and float((y.detach() - x).abs().max()) <= 0.025 + 1e-6
    assert torch.unique(torch.round(y.detach() / 0.05)).numel() <= 256
    # LSQ quantiser: trainable step; its explicit gradient equals autograd's
    lq = Q.LSQQuantizer(Q.QATConfig(bits=4, use_lsq=True)).init_from(x)
    assert lq.qmin() == -8 and lq.qmax() == 7 and lq.scale() == pytest.approx(float(2 * x.abs().mean() / math.sqrt(7)), rel=1e-5)
    out = lq(x)
    g = torch.randn_like(x)
    (out * g).sum().backward()
    assert float(lq.scale_param_tensor().grad) == pytest.approx(lq.compute_scale_grad(x, g), rel=1e-4)
    assert lq.quant_params().qmax == 7
    lq.set_scale(-1.0)
    assert lq.scale() == pytest.approx(1e-6)
    # KL calibration ignores a lone outlier that min / max calibration spends its range on
    data = torch.cat([torch.randn(20000), torch.tensor([40.0])])
    mm, kl = Q.MinMaxObserver(), Q.KLDivergenceObserver(bins=512)
    mm.observe(data), kl.observe(data[:10000]), kl.observe(data[10000:])
    assert kl.type() == "KLDivergence" and kl.calc_qparams(8).scale < 0.5 * mm.calc_qparams(8).scale
    bulk = data[:20000]
    err = lambda qp: float((qp.dequantize(qp.quantize(bulk)) - bulk).pow(2).mean())
    assert err(kl.calc_qparams(8)) < err(mm.calc_qparams(8))
    kl.reset()
    assert not kl.has_data() and float(kl.hist.sum()) == 0 and kl.calc_qparams(8).scale == 1.0
    assert Q.MovingAverageMinMaxObserver is Q.MovingAverageObserver
    ctx = Q.QATContext(Q.QATConfig(bits=4))
    assert ctx.maybe_quantize(x) is x and not ctx.enabled()
    ctx.enable()
    q = ctx.maybe_quantize(x)
    assert torch.unique(q).numel() <= 16 and torch.unique(ctx.maybe_quantize(x, Q.MinMaxObserver())).numel() <= 16
    asym = Q.fake_quantize_with_observer(x.abs().requires_grad_(True), Q.MinMaxObserver(), 4, False)
    assert torch.unique(asym.detach()).numel() <= 16 and asym.requires_grad
    step = torch.nn.Parameter(torch.tensor([0.2]))
    assert torch.unique(ctx.maybe_lsq_quantize(x, step).detach()).numel() <= 16
    ctx.disable()
    assert ctx.maybe_lsq_quantize(x, step) is x


def test_scalar_vq_family_residual_audio_codebook_and_ste_quantizer():
    from transformers_fusion_b200.quant import codec, qat as Q
    torch.manual_seed(0)
    w = torch.randn(1001).clamp(-1, 1)
    q8 = E.Q8VectorQuantizer()
    i8 = q8.quantize(w)
    assert i8.dtype == torch.uint8 and i8.numel() == 1001 and float((q8.dequantize(i8) - w).abs().max()) <= 1.0 / 255 + 1e-6
    assert q8.find_nearest(-1.0) == 0 and q8.find_nearest(1.0) == 255
    q4 = E.Q4VectorQuantizer()
    p4 = q4.quantize(w)
    assert p4.numel() == 501 and q4.dequantize(p4, 1001).shape == (1001,)
    e0 = float((q4.dequantize(p4, 1001) - w).pow(2).mean())
    assert int(p4[0]) & 0xF == q4.find_nearest(float(w[0])) and int(p4[0]) >> 4 == q4.find_nearest(float(w[1]))
    for _ in range(40):                                            # EMA moves the 16 entries to the data's cluster means
        q4.update_ema(w, q4.quantize(w), 1001)
    assert float((q4.dequantize(q4.quantize(w), 1001) - w).pow(2).mean()) < e0 and q4.codebook().dtype == torch.float16
    assert E.Q4VectorQuantizer.fp16_to_float(E.Q4VectorQuantizer.float_to_fp16(0.5)) == 0.5 and E.Q4VectorQuantizer.float_to_fp16(1.0) == 0x3C00
    with pytest.raises(ValueError):
        E.Q8VectorQuantizer([0.0, 1.0])
    # residual VQ: every added layer lowers the reconstruction error
    feats = torch.randn(2, 64, 8)
    ac = E.AudioCodebook(E.AudioCodebookConfig(num_quantizers=3, codebook_size=16, embedding_dim=8)).fit(feats, iters=5)
    idx = ac.encode(feats)
    assert idx.shape == (3, 2, 64) and len(ac.quantizers()) == 3 and ac.total_commitment_loss() > 0 and ac.total_codebook_loss() == 0.0
    errs = [float((ac.decode(idx[:k]) - feats).pow(2).mean()) for k in (1, 2, 3)]
    assert errs[0] > errs[1] > errs[2] and ac.decode(idx).shape == feats.shape
    ac.encode(feats, update=True)
    # straight-through quantisation to container formats
    st = Q.STEQuantizer("Q_4")
    assert st.target_format() == codec.parse_format("Q_4") and st.bits_for_format() == 4
    x = torch.randn(512, requires_grad=True)
    y = st(x)
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones(512)) and not torch.equal(y.detach(), x.detach())
    assert torch.allclose(y.detach(), Q.ste_roundtrip_(x.detach().clone(), "Q_4"))
    mixed = st.forward_mixed(x.detach(), ["Q_8", "Q_32"], 256)
    assert torch.equal(mixed[256:], x.detach()[256:]) and not torch.equal(mixed[:256], x.detach()[:256])
    with pytest.raises(ValueError):
        st.forward_mixed(x.detach(), ["Q_8"], 256)
    codes, sc = st.quantize_Q1(x.detach())
    assert set(torch.unique(codes).tolist()) <= {0, 1, 2} and sc > 0
    c4, s4 = st.quantize_quant(x.detach())
    assert int(c4.max()) <= 15 and float((((c4.float() - 8) * s4) - x.detach()).abs().max()) <= s4 / 2 + 1e-6
    cb = E.CodebookQ4()
    snapped = st.quantize_with_codebook(x.detach(), cb)
    assert torch.unique(snapped).numel() <= 16 and cb.trained
    assert torch.unique(st.fake_quantize_qat(x.detach())).numel() <= 15
    assert torch.unique(st.lsq_quantize(x.detach(), torch.tensor([0.3]))).numel() <= 16
    assert torch.unique(st.fake_quantize_with_observer(x.detach(), Q.MinMaxObserver())).numel() <= 16
