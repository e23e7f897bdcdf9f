"""Multimodal engine helpers: tokenising front ends, alignment / Perceiver training blocks, sensor preprocessing, fusion."""
import math

import pytest
import torch

from transformers_fusion_b200.engines import multimodal as E
from transformers_fusion_b200.models import multimodal as MM


def test_front_ends_shapes_and_content():
    img = torch.arange(3 * 32 * 48, dtype=torch.float32).view(3, 32, 48)
    tok = E.PatchEmbed(16, 768).embed(img)
    assert tok.shape == (2 * 3, 768) and torch.equal(tok[0, :16], img[0, 0, :16])            # first row of the first tile, channel 0
    assert E.PatchEmbed(16, 64).embed(img).shape == (6, 64) and E.PatchEmbed(16, 1000).embed(img).shape == (6, 1000)
    wav = torch.sin(torch.arange(1600.0) * 0.1).repeat(2, 1)
    fr = E.AudioFramer(400, 160, 400).frame(wav)
    assert fr.shape == ((1600 - 400) // 160 + 1, 400) and float(fr[:, 0].abs().max()) == 0.0  # Hann window starts at zero
    assert E.AudioFramer(400, 160, 128).frame(torch.ones(100)).shape == (1, 128)
    vid = torch.stack([torch.full((3, 4, 4), float(t)) for t in range(16)])
    clips = E.VideoSampler(4, 48).sample(vid)
    assert clips.shape == (4, 48) and torch.allclose(clips[:, 0], torch.tensor([1.5, 5.5, 9.5, 13.5]))
    assert E.VideoSampler(8, 48).sample(vid[:3]).shape == (3, 48)


def test_alignment_and_perceiver_training_blocks_learn():
    torch.manual_seed(0)
    a, b = torch.randn(16, 24), torch.randn(16, 12)
    at = E.AlignTrainer(MM.CrossModalAlignment(24, 12, 16), lr=2e-2)
    losses = [at.train_step(a, b) for _ in range(40)]
    assert losses[-1] < losses[0] - 0.5 and at.stats().steps == 40 and at.stats().tokens == 40 * 32 and at.stats().tok_per_sec > 0
    pt = E.PerceiverTrainer(MM.Perceiver(16, 4, 2), lr=1e-2)
    x, y = torch.randn(2, 10, 16), torch.randn(2, 4, 16)
    pl = [pt.train_step(x, None, y) for _ in range(60)]
    assert pl[-1] < 0.5 * pl[0] and pt.stats().last_loss == pytest.approx(pl[-1])
    from transformers_fusion_b200.tokenizer import ByteTokenizer
    mt = MM.MultiModalTokenizer(ByteTokenizer())
    assert E.TokProbe.roundtrip(ByteTokenizer(), "héllo wörld") == 0
    ids = E.TokProbe.image_ids(mt, torch.rand(3, 16, 16))
    aud = E.TokProbe.audio_ids(mt, torch.randn(800))
    # the code tokens sit between the modality's begin / end markers
    assert sum(i >= mt.image_base for i in ids) >= len(ids) - 2 > 0 and sum(i >= mt.audio_base for i in aud) >= len(aud) - 2 > 0


def test_sensor_preprocessing_and_fusion_math():
    S = E.Sensor3D
    pts = torch.tensor([[0.0, 0.0, 0.0], [1.0, 1.0, 1.0], [0.9, 0.9, 0.9], [0.1, 0.9, 0.1]])
    vox = S.voxelize(pts, 2, 2, 2)
    assert vox.sum() == 4 and vox[0, 0, 0] == 1 and vox[1, 1, 1] == 2 and vox[0, 1, 0] == 1
    plane = torch.arange(5.0)[None, :].repeat(4, 1) * 2.0                                    # depth rises by 2 per pixel in x
    n = S.depth_to_normals(plane)
    assert torch.allclose(n[2, 2], torch.tensor([-2.0, 0.0, 1.0]) / math.sqrt(5.0), atol=1e-6)
    t = S.normalize_thermal(torch.tensor([[10.0, 20.0], [30.0, 15.0]]))
    assert float(t.min()) == 0.0 and float(t.max()) == 1.0
    ms = torch.stack([torch.full((2, 2), 0.2), torch.full((2, 2), 0.6)])
    assert torch.allclose(S.spectral_index(ms, 0, 1), torch.full((2, 2), 0.5))
    base = torch.randn(1, 6, 6)
    hs = torch.cat([base * 3.0, base * -2.0, base * 0.5, torch.randn(2, 6, 6) * 0.01])
    pc = S.hs_pca3(hs)
    corr = torch.corrcoef(torch.stack([pc[0].reshape(-1), base.reshape(-1)]))[0, 1]
    assert pc.shape == (3, 6, 6) and abs(float(corr)) > 0.999 and pc[0].var() > 100 * pc[1].var()
    assert torch.allclose(S.sar_to_db(torch.tensor([1.0, 10.0, 0.1])), torch.tensor([0.0, 20.0, -20.0]), atol=1e-5)
    xyz = S.lidar_to_xyz(torch.tensor([2.0, 2.0]), torch.tensor([[0.0, 0.0], [math.pi / 2, math.pi / 6]]))
    assert torch.allclose(xyz, torch.tensor([[2.0, 0.0, 0.0], [0.0, math.sqrt(3.0), 1.0]]), atol=1e-6)
    assert torch.allclose(S.radar_speed(torch.tensor([[0.0, 0.0, 3.0, 4.0]])), torch.tensor([5.0]))
    tilt = S.imu_tilt(torch.tensor([[0.0, 0.0, 9.8, 0, 0, 0], [0.0, 9.8, 0.0, 0, 0, 0]]))
    assert torch.allclose(tilt, torch.tensor([[0.0, 0.0], [math.pi / 2, 0.0]]), atol=1e-6)
    loc = S.gps_local(torch.tensor([[48.001, 11.0], [48.0, 11.001]]), 48.0, 11.0)
    assert loc[0, 1] == pytest.approx(111.19, abs=0.2) and loc[1, 0] == pytest.approx(111.19 * math.cos(math.radians(48.0)), abs=0.2)
    Fm = E.FusionMath
    a, b = torch.randn(5, 8), torch.randn(7, 8)
    assert Fm.concat_last(a, a).shape == (5, 16)
    am = Fm.align_matrix(a, b)
    assert am.shape == (5, 7) and float(am.abs().max()) <= 1.0 + 1e-6 and torch.allclose(Fm.align_matrix(a, a).diagonal(), torch.ones(5), atol=1e-6)
    hi, lo = torch.full((2, 4), 10.0), torch.full((2, 4), -10.0)
    assert torch.allclose(Fm.gated_sum(hi, lo), hi, atol=1e-4) and torch.allclose(Fm.gated_sum(a, a), a)
    lat = torch.zeros(3, 8)
    step = Fm.perceiver_step(lat, b, heads=2)
    assert torch.allclose(step, b.mean(0).expand(3, 8), atol=1e-5)                           # zero queries: uniform attention = the mean
    assert E.modality_name(E.Modality.LIDAR) == "lidar" and E.NUM_MODALITIES == 26
