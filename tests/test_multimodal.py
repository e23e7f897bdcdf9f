import math

import pytest
import torch

from transformers_fusion_b200.models import multimodal as MM


def small_cfg():
    return MM.MultimodalEncoderConfig(image_patch_size=8, image_size=32, image_embed_dim=64, image_num_layers=1, image_num_heads=4,
                                      audio_n_mels=20, audio_embed_dim=32, audio_num_layers=1, audio_num_heads=4, text_vocab_size=100,
                                      text_embed_dim=48, text_max_len=32, text_num_layers=1, text_num_heads=4, shared_hidden=64,
                                      shared_num_heads=4, shared_num_layers=1, modality_dropout=0.0)


def test_towers_and_fusion_shapes_and_training():
    torch.manual_seed(0)
    m = MM.MultimodalCrossAttention(small_cfg())
    img, mel, ids = torch.randn(3, 3, 32, 32), torch.randn(3, 40, 20), torch.randint(0, 100, (3, 7))
    out = m(img, mel, ids)
    assert out["fused"].shape == (3, 17 + 10 + 7, 64) and out["spans"] == {"image": (0, 17), "audio": (17, 27), "text": (27, 34)}
    assert out["text_grounded"].shape == (3, 7, 64)
    loss = out["loss_image_text"] + out["loss_audio_text"]
    assert abs(float(out["loss_image_text"]) - math.log(3)) < 0.7
    loss.backward()
    assert m.vision.patch.proj.weight.grad is not None and m.text.emb.weight.grad is not None
    only_text = m(text_ids=ids)
    assert only_text["fused"].shape == (3, 7, 64) and "text_grounded" not in only_text
    # the alignment head learns to pair matching rows
    head = MM.ContrastiveAlignmentHead(16, 16, 8)
    a = torch.randn(6, 16)
    opt = torch.optim.Adam(head.parameters(), 1e-2)
    l0 = float(head(a, a + 0.01 * torch.randn(6, 16)))
    for _ in range(50):
        opt.zero_grad()
        l = head(a, a)
        l.backward()
        opt.step()
    assert float(l) < l0 and head.similarity(a, a).argmax(1).tolist() == list(range(6))


def test_mel_spectrogram_and_synthesis():
    sr = 8000
    t = torch.arange(sr).float() / sr
    mel = MM.MelSpectrogram(sr, 40, 256, 64)
    lo, hi = mel.compute(torch.sin(2 * math.pi * 300 * t)[None]), mel.compute(torch.sin(2 * math.pi * 2500 * t)[None])
    assert lo.shape[0] == 1 and lo.shape[2] == 40
    assert int(lo[0].mean(0).argmax()) < int(hi[0].mean(0).argmax())            # a higher tone lights a higher mel band
    fb = MM.MelSpectrogram.mel_filterbank(10, 64, 8000)
    assert fb.shape == (10, 33) and bool((fb >= 0).all()) and bool((fb.sum(1) > 0).all())
    wav = MM.AudioSynthesizer(mel, iters=4).synthesize(lo[0])
    assert wav.numel() > 7000 and torch.isfinite(wav).all()
    spec = torch.fft.rfft(wav[: 4096]).abs()
    assert abs(int(spec.argmax()) * sr / 4096 - 300) < 120                       # the reconstructed tone is where it was
    enc = MM.AudioTransformer(MM.AudioEncoderConfig(40, 32, 4, 1))
    assert MM.AudioFeatureExtractor(enc, mel).extract(torch.randn(2, 4000)).shape == (2, 32)


def test_perceiver_moe_fusion_tokenizer():
    torch.manual_seed(1)
    p = MM.Perceiver(32, 5, 4)
    assert p(torch.randn(2, 77, 32)).shape == (2, 5, 32)
    moe = MM.VisionTextMoE(32, 4)
    v, t = moe(torch.randn(2, 6, 32), torch.randn(2, 3, 32))
    assert v.shape == (2, 6, 32) and t.shape == (2, 3, 32) and float(moe.shared.last_aux) > 0
    am = MM.AllModalityMoE(32, 2)(image=torch.randn(1, 4, 32), audio=None, text=torch.randn(1, 2, 32))
    assert set(am) == {"image", "text"} and am["text"].shape == (1, 2, 32)
    for mode in ("concat", "gated", "cross_attention"):
        f = MM.MultimodalFusion(MM.FusionConfig(32, 4, mode))
        assert f(torch.randn(2, 5, 32), torch.randn(2, 9, 32)).shape == (2, 5, 32)
    tk = MM.MultiModalTokenizer(image_codes=16, audio_codes=8)
    ids = tk.encode("hi", [3, 15], [7])
    d = tk.decode(ids)
    assert d == {"text": "hi", "image_codes": [3, 15], "audio_codes": [7]} and max(ids) < tk.vocab_size and tk.BOI in ids


def test_task_heads():
    torch.manual_seed(2)
    vit = MM.VisionTransformer(MM.ViTConfig(32, 8, 3, 32, 4, 1, 64))
    img = torch.randn(2, 3, 32, 32)
    clf = MM.ImageNetClassifier(vit, 10)
    top = clf.classify(img, 3)
    assert len(top) == 2 and len(top[0]) == 3 and abs(sum(p for _, p in clf.classify(img, 10)[0]) - 1) < 1e-4
    assert MM.ctc_greedy_decode(torch.log(torch.tensor([[.1, .9, 0], [.1, .9, 0], [.9, .1, 0], [0, .1, .9], [0, .9, .1]]) + 1e-9)) == [1, 2, 1]
    asr = MM.SpeechRecognizer(MM.AudioTransformer(MM.AudioEncoderConfig(20, 32, 4, 1)), 12)
    mel = torch.randn(2, 40, 20)
    l = asr.loss(mel, torch.randint(1, 12, (2, 4)), torch.tensor([4, 3]))
    l.backward()
    assert torch.isfinite(l) and len(asr.transcribe(mel)) == 2
    ocr = MM.OCREngine(vit, 128)
    boxes = ocr.recognize(img)
    assert len(boxes) == 2 and boxes[0].w == 32 and isinstance(boxes[0].text, str)
    vid = MM.VideoUnderstanding(MM.VideoEncoder(vit, 1), 5)
    assert vid(torch.randn(2, 3, 3, 32, 32)).shape == (2, 5)
    cap = MM.ImageCaptioning(vit, 50, 32, 1, 4, 16)
    assert cap(img, torch.randint(0, 50, (2, 6))).shape == (2, 6, 50) and cap.caption(img, max_tokens=4).shape[1] <= 5
    txt = MM.TextEncoder(50, 32, 1, 4, 16)
    assert MM.VisualQA(vit, txt, 7, 32)(img, torch.randint(0, 50, (2, 5))).shape == (2, 7)
    t2i = MM.TextToImage(txt, num_codes=16, grid=2, dim=32, layers=1, heads=4, patch=4)
    assert t2i.generate(torch.randint(0, 50, (2, 5))).shape == (2, 3, 8, 8)
    assert MM.TextDecoder(50, 32, 1, 4, 16)(torch.randint(0, 50, (2, 5))).shape == (2, 5, 50)


def test_containers(tmp_path):
    im = MM.Image(torch.rand(3, 20, 30))
    assert im.resize(10, 12).data.shape == (3, 10, 12) and im.center_crop(16).data.shape == (3, 16, 16) and im.to_grayscale().data.shape == (1, 20, 30)
    im.save_ppm(str(tmp_path / "a.ppm"))
    back = MM.Image.load_ppm(str(tmp_path / "a.ppm"))
    assert back.data.shape == (3, 20, 30) and float((back.data - im.data).abs().max()) < 1 / 255 + 1e-6
    v = MM.Video(torch.rand(30, 3, 8, 8), 30.0)
    assert v.sample_uniform(5).frames.shape[0] == 5 and v.duration() == 1.0
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    se = MM.SentenceEmbedder(MM.TextEncoder(259, 32, 1, 4, 64), ByteTokenizer())
    assert se.embed(["a", "bb"]).shape == (2, 32) and se.similarity("same", "same") == pytest.approx(1.0, abs=1e-5)


@pytest.mark.gpu
def test_towers_on_device_kernels_match_torch_path():
    """bf16 on CUDA without autograd takes the GEMM / flash-attention kernels; with autograd it takes the torch path."""
    torch.manual_seed(0)
    vit = MM.VisionTransformer(MM.ViTConfig(32, 8, 3, 128, 2, 2, 256)).cuda().to(torch.bfloat16)
    img = torch.randn(2, 3, 32, 32, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        fast = vit(img, return_tokens=True).float()
    slow = vit(img.requires_grad_(), return_tokens=True).float().detach()
    assert (fast - slow).abs().max() / slow.abs().max() < 0.05
    txt = MM.TextEncoder(100, 128, 1, 2, 64).cuda().to(torch.bfloat16)
    ids = torch.randint(0, 100, (2, 33), device="cuda")
    with torch.no_grad():
        a = txt(ids).float()
    b = txt.emb.weight.requires_grad_() is not None and txt(ids).float().detach()
    assert (a - b).abs().max() / b.abs().max() < 0.05


def test_reference_named_multimodal_verbs(tmp_path):
    torch.manual_seed(1)
    cfg = small_cfg()
    m = MM.MultimodalCrossAttention(cfg).eval()
    img, mel, ids = torch.randn(2, 3, 32, 32), torch.randn(2, 40, 20), torch.randint(3, 100, (2, 6))
    # towers
    v = m.vision_encoder()
    assert v.encode(img).shape == (2, 64) and v.hidden_size() == 64 and v.is_initialized() and v.config() is v.cfg
    assert v.get_patch_features(img).shape == (2, 16, 64) and v.patch_embed(img).shape == (2, 16, 64)
    before = v.patch.proj.weight.clone()
    assert not torch.equal(v.init(5).patch.proj.weight, before)
    a = m.audio_encoder()
    assert a.encode(mel).shape == (2, 32) and a.n_mels() == 20 and a.d_model() == 32 and m.text_embedding().encode(ids).shape == (2, 48)
    # joint model
    assert m.encode_image(img).shape == (2, 64) and m.encode_audio(mel).shape == (2, 32) and m.encode_text(ids).shape == (2, 48)
    assert m.forward_text_image(ids, img).shape == (2, 6, 64) and m.forward_text_audio(ids, mel).shape == (2, 6, 64)
    assert m.add_image_tokens(img).shape == (2, 17, 64) and m.add_audio_tokens(mel).shape == (2, 10, 64) and m.add_text_tokens(ids).shape == (2, 6, 64)
    idx, sims = m.retrieve_images(ids[:1], torch.randn(5, 3, 32, 32), top_k=3)
    assert len(idx) == 3 and sims == sorted(sims, reverse=True)
    idx, _ = m.retrieve_text(img[:1], torch.randint(3, 100, (4, 6)), top_k=2)
    assert len(idx) == 2 and m.contrastive_head("audio_text") is m.align_at and m.config() is cfg
    cap = m.generate_caption(img[:1], max_tokens=4)
    ans = m.visual_question_answer(img[:1], ids[:1], max_tokens=3)
    assert 1 <= len(cap) <= 4 and 1 <= len(ans) <= 3 and all(0 <= t < 100 for t in cap + ans)
    # fusion encoder modes
    fe = m.fusion
    iv, av, tv = m.vision(img, return_tokens=True), m.audio(mel), m.text(ids)
    assert fe.fuse(iv, av, tv).shape == (2, 33, 64) and fe.fuse_late(iv, av, tv).shape == (2, 64)
    per = fe.get_per_modality_features(iv, None, tv)
    assert set(per) == {"image", "text"} and per["text"].shape == (2, 64)
    g = torch.Generator().manual_seed(0)
    drops = [fe.apply_modality_dropout({"image": iv, "audio": av, "text": tv}, 0.7, g) for _ in range(20)]
    assert all(any(t is not None for t in d.values()) for d in drops) and any(sum(t is None for t in d.values()) >= 1 for d in drops)
    # alignment head names
    head = MM.ContrastiveAlignmentHead(64, 48, 16)
    pa, pb = head.align_features(m.encode_image(img), m.encode_text(ids))
    assert torch.allclose(pa.norm(dim=-1), torch.ones(2), atol=1e-5) and head.project(m.encode_text(ids), "b").shape == (2, 16)
    clip, nce = head.compute_clip_loss(m.encode_image(img), m.encode_text(ids)), head.compute_infonce_loss(m.encode_image(img), m.encode_text(ids))
    assert clip > 0 and nce > 0
    head.set_temperature(0.5)
    assert head.get_temperature() == pytest.approx(0.5)
    # pairwise / weighted fusion
    fz = MM.MultimodalFusion(MM.FusionConfig(hidden=64, num_heads=4))
    vi, au, tx = torch.randn(2, 5, 64), torch.randn(2, 7, 64), torch.randn(2, 3, 64)
    assert fz.fuse_vision_text(vi, tx).shape == (2, 3, 64) and fz.fuse_audio_text(au, tx).shape == (2, 3, 64) and fz.fuse_vision_audio(vi, au).shape == (2, 5, 64)
    w = fz.compute_fusion_weights(vi, 3 * au, tx)
    assert abs(float(w.sum()) - 1) < 1e-6 and int(w.argmax()) == 1 and fz.fuse_weighted([vi, au, tx]).shape == (2, 64)
    assert fz.fuse_all(vi, au, tx).shape == (2, 3, 64) and [t.shape[1] for t in fz.fuse_all_multistream(vi, au, tx)] == [5, 7, 3]
    assert fz.param_count() > 0 and MM.ModalityProjection(8, 4).project_vision(torch.randn(2, 8)).shape == (2, 4)
    blk = MM.CrossAttentionBlock(MM.CrossAttentionLayerConfig(64, 4, 16))
    assert torch.allclose(blk.forward_self_attn(vi), blk(vi, vi))
    # tokenizer, containers
    tk = MM.MultiModalTokenizer(image_codes=64, audio_codes=32)
    pic = MM.Image(torch.linspace(0, 1, 3 * 16 * 16).view(3, 16, 16))
    ids_i = tk.encode_image(pic, grid=4)
    assert ids_i[0] == tk.BOI and ids_i[-1] == tk.EOI and len(ids_i) == 18 and tk.decode(ids_i)["image_codes"][-1] == 63
    ids_a = tk.encode_audio(torch.randn(50, 20), frames=8)
    assert len(tk.decode(ids_a)["audio_codes"]) == 8 and tk.image_token_id(3) == tk.image_base + 3 and tk.audio_token_id() == tk.audio_base
    assert (pic.channels(), pic.height(), pic.width(), pic.numel()) == (3, 16, 16, 768) and pic.to_tensor() is pic.data
    pic.save(str(tmp_path / "p.ppm"))
    assert torch.allclose(MM.Image.load(str(tmp_path / "p.ppm")).data, pic.data, atol=1 / 255)
    vid = MM.Video(torch.rand(3, 3, 8, 8))
    vid.save(str(tmp_path / "clip"))
    back = MM.Video.load(str(tmp_path / "clip"))
    assert back.num_frames() == 3 and (back.height(), back.width()) == (8, 8) and torch.allclose(back.frame(1).data, vid.frame(1).data, atol=1 / 255)
    # task heads
    vit = MM.VisionTransformer(MM.ViTConfig(32, 8, 3, 32, 4, 1, 64))
    clf = MM.ImageNetClassifier(vit, 10)
    ev = clf.evaluate(img, clf(img).argmax(-1))
    assert ev["top1"] == 1.0 and ev["top5"] == 1.0
    ve = MM.VideoEncoder(vit, 1)
    assert ve.encode(torch.randn(2, 3, 3, 32, 32)).shape == (2, 32) and ve.hidden_size() == 32
    desc = MM.VideoUnderstanding(ve, 4).describe(torch.randn(1, 3, 3, 32, 32), ["run", "jump", "sit", "wave"], 2)
    assert desc.count("(") == 2 and any(n in desc for n in ("run", "jump", "sit", "wave"))
    text = MM.TextEncoder(100, 32, 1, 4, 32)
    vqa = MM.VisualQA(vit, text, 3)
    assert vqa.answer(img, ids, ["yes", "no", "maybe"])[0] in ("yes", "no", "maybe") and len(vqa.answer(img, ids)) == 2
    assert len(MM.TextDecoder(100, 32, 1, 4, 32).decode([1, 2, 3], max_tokens=4)) == 4
    mel_t = MM.MelSpectrogram(16000, 20)
    assert mel_t.extract(torch.randn(1600)).shape[0] == 1 and mel_t.feature_length(1600) == 11 and mel_t.init(8000).sr == 8000
    fx = MM.AudioFeatureExtractor(MM.AudioTransformer(MM.AudioEncoderConfig(20, 32, 4, 1)))
    assert fx.init(16000).is_initialized()
    se = MM.SentenceEmbedder(text, type("T", (), {"encode": staticmethod(lambda s: [ord(c) % 100 for c in s])})())
    assert se.forward(["ab"]).shape == (1, 32) and se.hidden_size() == se.output_size() == 32
