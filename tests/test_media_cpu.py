"""Native media utilities: WAV parsing, resampling, log-mel spectrogram vs the Hugging Face Whisper extractor, images."""
import io
import struct
import wave

import numpy as np
import pytest

from tensorrt_edge_llm_b200.runtime import native as rt


def _wav_bytes(x, rate, channels=1, width=2):
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(channels)
        w.setsampwidth(width)
        w.setframerate(rate)
        pcm = (np.clip(x, -1, 1) * (2 ** (8 * width - 1) - 1)).astype({2: np.int16, 4: np.int32}[width])
        w.writeframes(np.repeat(pcm[:, None], channels, 1).tobytes())
    return buf.getvalue()


def test_wav_parse_and_resample():
    t = np.arange(8000) / 8000.0
    x = 0.5 * np.sin(2 * np.pi * 440 * t).astype(np.float32)
    for width in (2, 4):
        clip = rt.parse_wav(_wav_bytes(x, 8000, channels=2, width=width))
        assert clip.sample_rate == 8000 and clip.samples.shape == (8000,)
        assert np.abs(clip.samples - x).max() < 1e-3
    f32 = b"RIFF" + struct.pack("<I", 36 + 4 * len(x)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 3, 1, 8000, 32000, 4, 32) + b"data" + \
        struct.pack("<I", 4 * len(x)) + x.tobytes()
    assert np.array_equal(rt.parse_wav(f32).samples, x)
    y = rt.resample_linear(x, 8000, 16000)
    assert y.shape == (16000,) and np.abs(y[::2] - x).max() < 1e-6
    with pytest.raises(RuntimeError):
        rt.parse_wav(b"not a wave file at all")


def test_log_mel_matches_whisper_feature_extractor():
    from transformers import WhisperFeatureExtractor
    fe = WhisperFeatureExtractor(feature_size=128, sampling_rate=16000, hop_length=160, chunk_length=2, n_fft=400)
    rng = np.random.default_rng(0)
    t = np.arange(24000) / 16000.0
    x = (0.3 * np.sin(2 * np.pi * 300 * t) + 0.2 * np.sin(2 * np.pi * 2500 * t) + 0.05 * rng.standard_normal(t.shape)).astype(np.float32)
    want = fe(x, sampling_rate=16000, return_tensors="np")["input_features"][0]        # [128, 200]; the clip is cut to 2 s
    cfg = rt.MelConfig()
    cfg.pad_to_samples = 32000
    got = rt.log_mel_spectrogram(x, cfg)
    assert got.shape == want.shape == (128, 200)
    assert np.abs(got - want).max() < 2e-3
    fb = rt.mel_filterbank(cfg)
    assert fb.shape == (128, 201) and np.abs(fb - fe.mel_filters.T).max() < 1e-6


def test_images():
    rng = np.random.default_rng(1)
    px = rng.integers(0, 256, (6, 8, 3), dtype=np.uint8)
    ppm = b"P6\n# comment\n8 6\n255\n" + px.tobytes()
    im = rt.parse_image(ppm)
    assert (im.width, im.height, im.channels) == (8, 6, 3) and np.array_equal(im.pixels, px)
    row = (8 * 3 + 3) & ~3
    bmp = b"BM" + struct.pack("<IHHI", 54 + row * 6, 0, 0, 54) + struct.pack("<IiiHHIIiiII", 40, 8, 6, 1, 24, 0, row * 6, 0, 0, 0, 0)
    for y in range(5, -1, -1):
        bmp += px[y, :, ::-1].tobytes() + b"\0" * (row - 24)
    assert np.array_equal(rt.parse_image(bmp).pixels, px)
    grey = rt.parse_image(b"P5 2 2 255\n" + bytes([0, 50, 100, 200]))
    assert grey.channels == 3 and grey.pixels[1, 1].tolist() == [200, 200, 200]
    same = rt.resize_bilinear(im, 8, 6)
    assert np.array_equal(same.pixels, px)
    flat = rt.image_from_array(np.full((4, 4, 3), 77, np.uint8))
    assert (rt.resize_bicubic(flat, 9, 7).pixels == 77).all() and (rt.resize_bilinear(flat, 2, 3).pixels == 77).all()
    import torch
    up = rt.resize_bilinear(im, 16, 12).pixels.astype(np.float32)
    ref = torch.nn.functional.interpolate(torch.from_numpy(px).permute(2, 0, 1)[None].float(), size=(12, 16), mode="bilinear", align_corners=False)
    assert np.abs(up - ref[0].permute(1, 2, 0).numpy()).max() <= 0.51
    chw = rt.normalize_chw(im, [0.5, 0.5, 0.5], [0.25, 0.25, 0.25])
    assert chw.shape == (3, 6, 8) and np.allclose(chw[1, 2, 3], (px[2, 3, 1] / 255 - 0.5) / 0.25, atol=1e-6)
    assert rt.smart_resize(1000, 700, 28, 56 * 56, 28 * 28 * 256) == (504, 364) or all(v % 28 == 0 for v in rt.smart_resize(1000, 700, 28, 3136, 200704))
    h, w = rt.smart_resize(20, 30, 28, 3136, 200704)
    assert h % 28 == 0 and w % 28 == 0 and h * w >= 3136
    with pytest.raises(RuntimeError):
        rt.parse_image(b"\x89PNG....")
