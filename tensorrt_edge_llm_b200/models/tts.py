"""Speech generation models: Talker, CodePredictor, the text front end and the Code2Wav vocoder.

An audio frame is ``num_code_groups`` residual-VQ codes.  The **Talker** (a Qwen3-style decoder over codec tokens) emits
the first code of each frame and hands its final hidden state on; the **CodePredictor** (a small decoder with one LM
head and one codec embedding per remaining codebook) emits the other codes of that frame, one pass each; the sum of the
frame's codec embeddings plus the next text row is the Talker's next input.  **Code2Wav** turns the code matrix into a
waveform: codebook lookups summed over the quantisers, a causal convolution, a sliding-window transformer, transposed
convolution + ConvNeXt upsampling stages, then decoder blocks of SnakeBeta activations, transposed convolutions and
dilated residual units; every stage is causal, so a chunk decoded with enough left context equals the same span of a
full decode.

Parity: ``tensorrt_edgellm/models/qwen3_tts/modeling_qwen3_tts_talker.py`` (hidden states beside the logits),
``modeling_code_predictor.py`` (stacked heads picked by index, fp32 ``silu(gate) * up`` and down projection,
``small_to_mtp_projection``), ``modeling_qwen3_tts_text.py`` (text embedding + projection MLP),
``modeling_qwen3_tts_code2wav.py`` (config fields :46-71, causal convolutions, SnakeBeta, decoder blocks); the frame
loop that drives them is ``cpp/runtime/qwen3OmniTTSRuntime.cpp`` (``runtime/tts.py`` here).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..config import ModelConfig
from ..model import register_model
from ..ops.meta import StepMeta
from .default import CausalLM


# ---- configuration ---------------------------------------------------------------------------------------------------

@dataclass
class Code2WavConfig:
    codebook_size: int = 2048
    codebook_dim: int = 512
    hidden_size: int = 1024
    latent_dim: int = 1024
    num_hidden_layers: int = 8
    num_attention_heads: int = 16
    head_dim: Optional[int] = None
    intermediate_size: int = 3072
    sliding_window: int = 72
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    layer_scale_initial_scale: float = 0.01
    num_quantizers: int = 16
    num_semantic_quantizers: int = 1
    upsampling_ratios: Tuple[int, ...] = (2, 2)
    upsample_rates: Tuple[int, ...] = (8, 5, 4, 3)
    decoder_dim: int = 1536
    sample_rate: int = 24000

    def __post_init__(self):
        self.upsampling_ratios = tuple(self.upsampling_ratios)
        self.upsample_rates = tuple(self.upsample_rates)
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    @property
    def samples_per_frame(self) -> int:
        return math.prod(self.upsampling_ratios) * math.prod(self.upsample_rates)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Code2WavConfig":
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})


@dataclass
class TTSConfig:
    """Everything the frame loop needs beside the three models' own configurations."""
    num_code_groups: int = 16
    codebook_size: int = 2048               # codec ids below this are audio codes; the talker's ids above it are control tokens
    text_vocab_size: int = 151936
    text_hidden_size: int = 2048
    codec_bos_id: int = 2149
    codec_eos_id: int = 2150
    codec_pad_id: int = 2148
    codec_nothink_id: int = 2155
    codec_think_id: int = 2154
    codec_think_bos_id: int = 2156
    codec_think_eos_id: int = 2157
    tts_bos_token_id: int = 151672
    tts_eos_token_id: int = 151673
    tts_pad_token_id: int = 151671
    role_prefix_tokens: int = 3             # "<|im_start|>assistant\n"
    suffix_tokens: int = 5                  # "<|im_end|>\n<|im_start|>assistant\n"
    role_prefix_ids: List[int] = field(default_factory=list)          # the template's token ids, for callers that hold bare text ids
    suffix_ids: List[int] = field(default_factory=list)
    speakers: Dict[str, int] = field(default_factory=dict)            # name → codec id of the speaker row
    languages: Dict[str, int] = field(default_factory=dict)           # name → codec id of the language row
    speaker_dialects: Dict[str, str] = field(default_factory=dict)    # speaker → language it switches on by itself
    default_speaker: str = ""
    tts_model_type: str = "custom_voice"

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TTSConfig":
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

    def language_id(self, language: Optional[str], speaker: Optional[str]) -> Optional[int]:
        """The codec id of the language row, or None for the no-language prompt.  A dialect speaker switches its dialect
        on when the request says ``auto`` or ``chinese``; an unknown name falls back to ``auto``."""
        lang = (language or "auto").lower()
        dialect = self.speaker_dialects.get((speaker or "").lower())
        if dialect and lang in ("auto", "chinese"):
            lang = dialect
        return self.languages.get(lang) if lang != "auto" else None


# ---- talker and code predictor ---------------------------------------------------------------------------------------

@register_model("qwen3_tts_talker", "qwen3_omni_talker")
class TalkerCausalLM(CausalLM):
    """A decoder over codec tokens whose step also leaves the final-norm hidden state of every logits row in
    ``last_hidden``: the CodePredictor's first input row."""

    def __init__(self, cfg: ModelConfig, comm=None):
        super().__init__(cfg, comm)
        self.last_hidden: Optional[torch.Tensor] = None

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        if key.startswith("code_predictor.") or key.startswith(("text_embedding.", "text_projection.")):
            return None                                            # own modules, loaded by their own classes
        return key.replace("model.codec_embedding.", "model.embed_tokens.").replace("codec_head.", "lm_head.")

    def forward(self, ids, meta: StepMeta, kv_cache, inputs_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.hidden_states(ids, meta, kv_cache, inputs_embeds)
        self.last_hidden = x if meta.logits_idx.numel() == x.shape[0] else x.index_select(0, meta.logits_idx.long())
        return self.lm_head(self.last_hidden)


def _fp32_guard_mlp_forward(self, x):
    """SwiGLU whose product and down projection run in fp32: the CodePredictor's activations are large enough that a
    16-bit product loses the low bits that decide the codec's end-of-stream prediction."""
    gate, up = self.gate_up_proj(x).float().chunk(2, dim=-1)
    return F.linear(F.silu(gate) * up, self.down_proj.weight.float()).to(x.dtype)


@register_model("qwen3_tts_code_predictor", "qwen3_omni_code_predictor")
class CodePredictorCausalLM(CausalLM):
    """``num_code_groups - 1`` heads and codec embeddings around one small decoder.  ``forward`` returns final-norm hidden
    rows; ``head_logits(hidden, j)`` scores them with head ``j``; ``embed(j, codes)`` looks codes up in table ``j`` (rows
    of the Talker's width) and ``project`` brings Talker-width rows to this model's width."""

    def __init__(self, cfg: ModelConfig, comm=None, num_code_groups: int = 16, talker_hidden_size: Optional[int] = None):
        super().__init__(cfg, comm)
        n = num_code_groups - 1
        th = talker_hidden_size or cfg.hidden_size
        dt = cfg.compute_dtype
        self.num_heads = n
        self.lm_heads = nn.Parameter(torch.zeros(n, cfg.vocab_size, cfg.hidden_size, dtype=dt), requires_grad=False)
        self.codec_embeddings = nn.Parameter(torch.zeros(n, cfg.vocab_size, th, dtype=dt), requires_grad=False)
        self.small_to_mtp_projection = nn.Linear(th, cfg.hidden_size, bias=True, dtype=dt) if th != cfg.hidden_size else None
        if cfg.compute_dtype != torch.float32:
            import types
            for layer in self.model.layers:
                if not torch.is_floating_point(getattr(layer.mlp.down_proj, "weight", torch.zeros(0, dtype=torch.uint8))):
                    raise ValueError("the CodePredictor's down_proj must stay unquantised: its product runs in fp32")
                layer.mlp.forward = types.MethodType(_fp32_guard_mlp_forward, layer.mlp)

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        return key

    def load_stacked(self, heads: Sequence[torch.Tensor], embeddings: Sequence[torch.Tensor]) -> None:
        """Stack the checkpoint's per-codebook ``lm_head.{j}.weight`` / ``model.codec_embedding.{j}.weight`` tensors."""
        with torch.no_grad():
            self.lm_heads.copy_(torch.stack([h.to(self.lm_heads.dtype) for h in heads]))
            self.codec_embeddings.copy_(torch.stack([e.to(self.codec_embeddings.dtype) for e in embeddings]))

    def project(self, rows: torch.Tensor) -> torch.Tensor:
        return rows if self.small_to_mtp_projection is None else self.small_to_mtp_projection(rows)

    def embed(self, j: int, codes: torch.Tensor) -> torch.Tensor:
        return self.codec_embeddings[j].index_select(0, codes.long().reshape(-1))

    def head_logits(self, hidden: torch.Tensor, j: int) -> torch.Tensor:
        return (hidden @ self.lm_heads[j].t()).float()

    def forward(self, ids, meta: StepMeta, kv_cache, inputs_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.hidden_states(ids, meta, kv_cache, inputs_embeds)
        return x if meta.logits_idx.numel() == x.shape[0] else x.index_select(0, meta.logits_idx.long())


class TextFrontEnd(nn.Module):
    """Text token → Talker input row: the text embedding table followed by a two-layer projection (biases, SiLU)."""

    def __init__(self, vocab_size: int, text_hidden: int, hidden: int, dtype=torch.float32):
        super().__init__()
        self.text_embedding = nn.Embedding(vocab_size, text_hidden, dtype=dtype)
        self.fc1 = nn.Linear(text_hidden, text_hidden, bias=True, dtype=dtype)
        self.fc2 = nn.Linear(text_hidden, hidden, bias=True, dtype=dtype)

    @staticmethod
    def checkpoint_key_remap(key: str) -> Optional[str]:
        for src, dst in (("text_projection.linear_fc1.", "fc1."), ("text_projection.linear_fc2.", "fc2."), ("model.text_embedding.", "text_embedding.")):
            if key.startswith(src):
                return dst + key[len(src):]
        return key if key.startswith(("text_embedding.", "fc1.", "fc2.")) else None

    @torch.no_grad()
    def forward(self, ids) -> torch.Tensor:
        ids = torch.as_tensor(ids, dtype=torch.long, device=self.text_embedding.weight.device).reshape(-1)
        return self.fc2(F.silu(self.fc1(self.text_embedding(ids))))


# ---- vocoder ---------------------------------------------------------------------------------------------------------

class CausalConv1d(nn.Module):
    """Convolution padded on the left only (``(k - 1) · dilation - (stride - 1)`` samples), so sample ``t`` of the output
    reads inputs up to ``t`` and nothing later."""

    def __init__(self, cin: int, cout: int, kernel: int, dilation: int = 1, stride: int = 1, groups: int = 1):
        super().__init__()
        self.conv = nn.Conv1d(cin, cout, kernel, stride=stride, dilation=dilation, groups=groups)
        self.left = (kernel - 1) * dilation - (stride - 1)

    def forward(self, x):
        return self.conv(F.pad(x, (self.left, 0)))


class CausalTransConv1d(nn.Module):
    """Transposed convolution that keeps ``stride`` outputs per input: the ``kernel - stride`` extra samples at the right
    end, which would read like a look-ahead, are cut."""

    def __init__(self, cin: int, cout: int, kernel: int, stride: int):
        super().__init__()
        self.conv = nn.ConvTranspose1d(cin, cout, kernel, stride=stride)
        self.cut = kernel - stride

    def forward(self, x):
        y = self.conv(x)
        return y[..., : y.shape[-1] - self.cut] if self.cut > 0 else y


class SnakeBeta(nn.Module):
    """``x + sin²(α x) / β`` with per-channel α, β stored as logarithms."""

    def __init__(self, channels: int):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(channels))
        self.beta = nn.Parameter(torch.zeros(channels))

    def forward(self, x):
        a = self.alpha.exp()[None, :, None]
        b = self.beta.exp()[None, :, None]
        return x + torch.sin(x * a).pow(2) / (b + 1e-9)


class ConvNeXtBlock(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.dwconv = CausalConv1d(dim, dim, 7, groups=dim)
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.pwconv1 = nn.Linear(dim, 4 * dim)
        self.pwconv2 = nn.Linear(4 * dim, dim)
        self.gamma = nn.Parameter(torch.full((dim,), 1e-6))

    def forward(self, x):
        y = self.dwconv(x).transpose(1, 2)
        y = self.pwconv2(F.gelu(self.pwconv1(self.norm(y)))) * self.gamma
        return x + y.transpose(1, 2)


class ResidualUnit(nn.Module):
    def __init__(self, dim: int, dilation: int):
        super().__init__()
        self.act1, self.conv1 = SnakeBeta(dim), CausalConv1d(dim, dim, 7, dilation=dilation)
        self.act2, self.conv2 = SnakeBeta(dim), CausalConv1d(dim, dim, 1)

    def forward(self, x):
        return x + self.conv2(self.act2(self.conv1(self.act1(x))))


class DecoderBlock(nn.Module):
    def __init__(self, cin: int, cout: int, rate: int):
        super().__init__()
        self.act = SnakeBeta(cin)
        self.up = CausalTransConv1d(cin, cout, 2 * rate, rate)
        self.units = nn.ModuleList([ResidualUnit(cout, d) for d in (1, 3, 9)])

    def forward(self, x):
        x = self.up(self.act(x))
        for u in self.units:
            x = u(x)
        return x


class _TorchRMSNorm(nn.Module):
    """RMSNorm in plain torch ops: the vocoder runs in fp32, which the decoder stack's 16-bit norm kernel does not take."""

    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


class _SlidingLayer(nn.Module):
    def __init__(self, c: Code2WavConfig):
        super().__init__()
        h, d, nh = c.hidden_size, c.head_dim, c.num_attention_heads
        self.nh, self.d = nh, d
        self.input_layernorm = _TorchRMSNorm(h, c.rms_norm_eps)
        self.post_attention_layernorm = _TorchRMSNorm(h, c.rms_norm_eps)
        self.q_proj, self.k_proj, self.v_proj = (nn.Linear(h, nh * d, bias=False) for _ in range(3))
        self.o_proj = nn.Linear(nh * d, h, bias=False)
        self.gate_proj, self.up_proj = nn.Linear(h, c.intermediate_size, bias=False), nn.Linear(h, c.intermediate_size, bias=False)
        self.down_proj = nn.Linear(c.intermediate_size, h, bias=False)
        self.attn_scale = nn.Parameter(torch.full((h,), c.layer_scale_initial_scale))
        self.mlp_scale = nn.Parameter(torch.full((h,), c.layer_scale_initial_scale))

    def forward(self, x, cos, sin, mask):
        b, t, _ = x.shape
        y = self.input_layernorm(x)
        q, k, v = (p(y).view(b, t, self.nh, self.d).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))

        def rot(u):
            u1, u2 = u[..., : self.d // 2], u[..., self.d // 2:]
            return torch.cat((u1 * cos - u2 * sin, u2 * cos + u1 * sin), dim=-1)

        a = F.scaled_dot_product_attention(rot(q), rot(k), v, attn_mask=mask)
        x = x + self.o_proj(a.transpose(1, 2).reshape(b, t, -1)) * self.attn_scale
        y = self.post_attention_layernorm(x)
        return x + self.down_proj(F.silu(self.gate_proj(y)) * self.up_proj(y)) * self.mlp_scale


class Code2Wav(nn.Module):
    """``forward(codes [B, G, F])`` → waveform ``[B, F · samples_per_frame]`` in [-1, 1] (fp32)."""

    def __init__(self, c: Code2WavConfig):
        super().__init__()
        self.cfg = c
        # one table per quantiser; the first ``num_semantic_quantizers`` and the rest have an output projection each
        self.codebooks = nn.Parameter(torch.zeros(c.num_quantizers, c.codebook_size, c.codebook_dim), requires_grad=False)
        self.semantic_proj = nn.Conv1d(c.codebook_dim, c.latent_dim, 1, bias=False)
        self.acoustic_proj = nn.Conv1d(c.codebook_dim, c.latent_dim, 1, bias=False)
        self.pre_conv = CausalConv1d(c.latent_dim, c.hidden_size, 3)
        self.layers = nn.ModuleList([_SlidingLayer(c) for _ in range(c.num_hidden_layers)])
        self.norm = _TorchRMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_proj = nn.Linear(c.hidden_size, c.latent_dim)
        self.upsample = nn.ModuleList([nn.Sequential(CausalTransConv1d(c.latent_dim, c.latent_dim, r, r), ConvNeXtBlock(c.latent_dim))
                                       for r in c.upsampling_ratios])
        dims = [c.decoder_dim // (2 ** i) for i in range(len(c.upsample_rates) + 1)]
        self.decoder_in = CausalConv1d(c.latent_dim, dims[0], 7)
        self.blocks = nn.ModuleList([DecoderBlock(dims[i], dims[i + 1], r) for i, r in enumerate(c.upsample_rates)])
        self.final_act = SnakeBeta(dims[-1])
        self.final_conv = CausalConv1d(dims[-1], 1, 7)

    def context_frames(self) -> int:
        """Left context (frames) after which a chunk's samples no longer depend on anything earlier: the transformer's
        reach (each layer looks ``sliding_window - 1`` frames back) plus the reach of every convolution, each counted in
        frames at the sample rate it runs at."""
        c = self.cfg
        reach = float(c.num_hidden_layers * (c.sliding_window - 1) + 2)          # transformer + the k=3 convolution before it
        rate = 1
        for r in c.upsampling_ratios:
            rate *= r
            reach += 6.0 / rate                                                  # ConvNeXt's k=7 depthwise convolution
        reach += 6.0 / rate                                                      # the decoder's k=7 input convolution
        for r in c.upsample_rates:
            reach += 1.0 / rate                                                  # a transposed convolution of kernel 2·stride reads two inputs
            rate *= r
            reach += 6.0 * (1 + 3 + 9) / rate                                    # three dilated k=7 residual units
        reach += 6.0 / rate                                                      # the final k=7 convolution
        return int(math.ceil(reach)) + 1

    @torch.no_grad()
    def forward(self, codes: torch.Tensor) -> torch.Tensor:
        # full-precision convolutions on the device too: with TF32 a chunk and the full decode pick different algorithms and
        # their samples drift apart by more than a 16-bit PCM step
        with torch.backends.cudnn.flags(enabled=True, benchmark=False, deterministic=False, allow_tf32=False):
            return self._forward(codes)

    def _forward(self, codes: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        codes = codes.long().clamp_(0, c.codebook_size - 1)
        b, g, t = codes.shape
        if g != c.num_quantizers:
            raise ValueError(f"Code2Wav expects {c.num_quantizers} codes per frame, got {g}")
        emb = torch.stack([self.codebooks[q].index_select(0, codes[:, q].reshape(-1)).view(b, t, -1) for q in range(g)], dim=1)   # [B, G, T, cd]
        ns = c.num_semantic_quantizers
        x = self.semantic_proj(emb[:, :ns].sum(1).transpose(1, 2)) + self.acoustic_proj(emb[:, ns:].sum(1).transpose(1, 2))
        x = self.pre_conv(x).transpose(1, 2)                                                                 # [B, T, H]
        pos = torch.arange(t, device=x.device, dtype=torch.float32)
        inv = c.rope_theta ** (-torch.arange(0, c.head_dim, 2, device=x.device, dtype=torch.float32) / c.head_dim)
        ang = pos[:, None] * inv[None, :]
        cos, sin = ang.cos()[None, None], ang.sin()[None, None]
        i = torch.arange(t, device=x.device)
        mask = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - c.sliding_window)
        for layer in self.layers:
            x = layer(x, cos, sin, mask)
        x = self.post_proj(self.norm(x)).transpose(1, 2)               # [B, latent, T]
        for up in self.upsample:
            x = up(x)
        x = self.decoder_in(x)
        for blk in self.blocks:
            x = blk(x)
        return self.final_conv(self.final_act(x)).squeeze(1).clamp(-1.0, 1.0)

    @torch.no_grad()
    def decode_chunk(self, codes: torch.Tensor, start: int, end: int) -> torch.Tensor:
        """Samples of frames ``[start, end)`` of ``codes [G, F]``, decoded with the left context the stack can see."""
        lo = max(0, start - self.context_frames())
        wav = self.forward(codes[None, :, lo:end])[0]
        return wav[(start - lo) * self.cfg.samples_per_frame:]


def pcm16_bytes(wav: torch.Tensor) -> bytes:
    """Float samples in [-1, 1] → little-endian 16-bit PCM."""
    return (wav.detach().float().clamp(-1, 1) * 32767.0).round().to(torch.int16).cpu().numpy().astype("<i2").tobytes()


def wav_file_bytes(pcm16: bytes, sample_rate: int, channels: int = 1) -> bytes:
    """A RIFF/WAVE container around 16-bit PCM."""
    import struct
    hdr = b"RIFF" + struct.pack("<I", 36 + len(pcm16)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, channels, sample_rate,
                                                                                  sample_rate * channels * 2, channels * 2, 16)
    return hdr + b"data" + struct.pack("<I", len(pcm16)) + pcm16
