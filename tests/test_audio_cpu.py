"""Audio encoder vs the Hugging Face Whisper encoder (same random weights), and the waveform → embedding-rows path."""
import numpy as np
import torch

from tensorrt_edge_llm_b200.models.audio import AudioConfig, AudioEncoder, audio_features, sinusoid_positions


def test_matches_hf_whisper_encoder():
    from transformers import WhisperConfig
    from transformers.models.whisper.modeling_whisper import WhisperEncoder
    hc = WhisperConfig(num_mel_bins=16, d_model=128, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=256, max_source_positions=50,
                       dropout=0.0, attention_dropout=0.0, activation_dropout=0.0)
    torch.manual_seed(0)
    ref = WhisperEncoder(hc).eval().float()
    enc = AudioEncoder(AudioConfig(n_mels=16, hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                                   max_source_positions=50, avg_pool=1, dtype="float32"))
    enc.load_hf_state_dict(ref.state_dict())
    assert torch.allclose(enc.embed_positions, sinusoid_positions(50, 128), atol=1e-6)
    mel = torch.randn(2, 16, 100)
    with torch.no_grad():
        want = ref(mel).last_hidden_state                      # [2, 50, 128]
    got = enc(mel).view(2, 50, 128)
    assert (got - want).abs().max() < 2e-4


def test_waveform_to_projected_rows():
    t = np.arange(16000) / 16000.0
    feats = audio_features(0.4 * np.sin(2 * np.pi * 220 * t), 16000, n_mels=16, chunk_seconds=1)
    assert feats.shape == (1, 16, 100)
    enc = AudioEncoder(AudioConfig(n_mels=16, hidden_size=128, num_hidden_layers=1, num_attention_heads=2, intermediate_size=256,
                                   max_source_positions=50, avg_pool=2, out_hidden_size=96, dtype="float32")).random_init(1)
    rows = enc(feats)
    assert rows.shape == (25, 96) and torch.isfinite(rows).all()
    half = audio_features(0.4 * np.sin(2 * np.pi * 220 * t[::2]), 8000, n_mels=16, chunk_seconds=1)      # resampled on the way in
    assert half.shape == feats.shape and (half - feats).abs().mean() < 0.05
