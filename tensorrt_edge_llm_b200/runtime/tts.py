"""Speech generation runtime: Talker + CodePredictor frame loop and the Code2Wav vocoder behind one ``TTS`` front end.

One request: the text becomes a Talker prefill (role rows, a codec prefix of control / language / speaker rows summed with
``tts_pad`` … ``tts_bos`` text rows, the first text row on ``codec_bos``); the rest of the text is fed one row per decode
step ("trailing text"), then ``tts_eos``, then ``tts_pad``.  Every Talker step samples the first code of a frame (with a
repetition penalty over the codes already emitted and every control id but end-of-stream masked); the CodePredictor then
starts from two rows (the Talker's hidden state, the first code's embedding) and emits the remaining codes one pass
each, code ``j + 1`` from head ``j``.  The frame's embeddings summed, plus the next trailing row, is the next Talker
input.  Codes stream to the vocoder in chunks as they are produced; each chunk is decoded with the left context the
vocoder can see, so the concatenated chunks equal one decode of the whole matrix.

Parity: ``cpp/runtime/qwen3OmniTTSRuntime.{h,cpp}`` (``runTalkerGenerationLoop``, ``PerBatchTalkerState``,
``computeResidualConnection``, the CodePredictor prefill / step pair, ``PerBatchStreamingHandler`` chunks),
``examples/cpp/qwen3_tts_inference.cpp`` and the guide ``docs/source/user_guide/examples/tts.md`` (request file keys:
``talker_temperature``, ``talker_top_k``, ``talker_top_p``, ``repetition_penalty``, ``max_audio_length``, ``speaker``,
``language``), Python ``TTS`` / nanobind ``TTSRuntime`` (``python/nanobind/bindings.cpp:559-590``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..config import ModelConfig, tiny_llama_config
from ..models.tts import (Code2Wav, Code2WavConfig, CodePredictorCausalLM, TalkerCausalLM, TextFrontEnd, TTSConfig, pcm16_bytes,
                          wav_file_bytes)
from .kv_cache import KVCacheManager
from .runner import ModelRunner, SamplingParams

TTS_CONFIG_NAME = "tts_config.json"


@dataclass
class TTSSampling:
    talker_temperature: float = 0.9
    talker_top_k: int = 50
    talker_top_p: float = 1.0
    repetition_penalty: float = 1.05
    predictor_temperature: float = 0.9
    predictor_top_k: int = 50
    predictor_top_p: float = 1.0
    max_audio_length: int = 4096            # codec frames
    seed: int = 42
    cp_spec_verify_size: int = 0            # CodePredictor head speculation: one committed depth + N-1 drafted ones per pass (0 = off, 2..8)

    @classmethod
    def from_dict(cls, d: Dict) -> "TTSSampling":
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})


@dataclass
class TTSResult:
    codes: torch.Tensor                     # [frames, num_code_groups] int32
    waveform: torch.Tensor                  # [samples] fp32 in [-1, 1]
    sample_rate: int
    finish_reason: str                      # "eos" | "length"
    talker_steps: int = 0
    predictor_steps: int = 0
    chunks: int = 0

    @property
    def frames(self) -> int:
        return int(self.codes.shape[0])

    @property
    def pcm16(self) -> bytes:
        return pcm16_bytes(self.waveform)

    def wav_bytes(self) -> bytes:
        return wav_file_bytes(self.pcm16, self.sample_rate)


class TTSRuntime:
    """Owns the three models, their KV pools and the frame loop.  One request at a time (seat 0 of each pool)."""

    def __init__(self, cfg: TTSConfig, talker: TalkerCausalLM, predictor: CodePredictorCausalLM, front: TextFrontEnd, code2wav: Code2Wav,
                 tokenizer=None, device="cpu", max_seq_len: int = 4096, page_size: int = 0):
        self.cfg, self.front, self.code2wav, self.tokenizer = cfg, front, code2wav, tokenizer
        self.device = torch.device(device)
        page_size = page_size or (64 if self.device.type == "cuda" else 16)      # the device attention kernels take 64- or 128-token pages
        pages = (max_seq_len + page_size - 1) // page_size + 1
        self.talker = ModelRunner(talker, KVCacheManager(talker.cfg, num_pages=pages, page_size=page_size, max_seats=1, max_pages_per_seq=pages,
                                                         device=self.device), device=self.device)
        cp_pages = (cfg.num_code_groups + 1 + page_size - 1) // page_size + 1
        self.predictor = ModelRunner(predictor, KVCacheManager(predictor.cfg, num_pages=cp_pages, page_size=page_size, max_seats=1,
                                                               max_pages_per_seq=cp_pages, device=self.device), device=self.device)
        self.max_seq_len = max_seq_len
        if predictor.num_heads != cfg.num_code_groups - 1:
            raise ValueError("the CodePredictor has one head per codebook after the first")
        if code2wav.cfg.num_quantizers != cfg.num_code_groups:
            raise ValueError("the vocoder's quantiser count differs from the frame width")

    # ---- prompt --------------------------------------------------------------------------------------------------------
    def voices(self) -> List[str]:
        return sorted(self.cfg.speakers)

    def tokenize(self, text: str) -> List[int]:
        if self.tokenizer is None:
            raise ValueError("this runtime was loaded without a tokenizer: pass token ids")
        return list(self.tokenizer.encode(f"<|im_start|>assistant\n{text}<|im_end|>\n<|im_start|>assistant\n"))

    def template_ids(self, text_ids: Sequence[int]) -> List[int]:
        """Bare text token ids (what a text decoder upstream produced) wrapped in the speech prompt's role prefix and suffix."""
        c = self.cfg
        if len(c.role_prefix_ids) != c.role_prefix_tokens or len(c.suffix_ids) != c.suffix_tokens:
            raise ValueError("this pipeline's configuration does not carry the template's token ids (role_prefix_ids / suffix_ids)")
        return list(c.role_prefix_ids) + [int(t) for t in text_ids] + list(c.suffix_ids)

    def _codec_rows(self, ids: Sequence[int]) -> torch.Tensor:
        return self.talker.embed_tokens(list(ids)).float()

    @torch.no_grad()
    def build_prefill(self, text_ids: Sequence[int], speaker: Optional[str] = None, language: Optional[str] = None):
        """``text_ids`` is the templated text (role prefix, text, suffix).  Returns ``(prefill rows [T, H], trailing rows
        [N, H], tts_pad row [1, H])``."""
        c = self.cfg
        text_ids = list(text_ids)
        if len(text_ids) < c.role_prefix_tokens + 1 + c.suffix_tokens:
            raise ValueError("the templated text is shorter than its role prefix, one text token and the suffix")
        name = (speaker or c.default_speaker or "").lower()
        if name and name not in c.speakers:
            raise ValueError(f"unknown speaker {speaker!r}; available: {self.voices()}")
        special = self.front([c.tts_bos_token_id, c.tts_eos_token_id, c.tts_pad_token_id]).float()
        tts_bos, tts_eos, tts_pad = special[0:1], special[1:2], special[2:3]
        lang = c.language_id(language, name)
        prefix = [c.codec_nothink_id, c.codec_think_bos_id, c.codec_think_eos_id] if lang is None else \
            [c.codec_think_id, c.codec_think_bos_id, lang, c.codec_think_eos_id]
        if name:
            prefix.append(c.speakers[name])
        codec = self._codec_rows(prefix + [c.codec_pad_id, c.codec_bos_id])                     # [L, H]
        text_side = torch.cat([tts_pad.expand(codec.shape[0] - 2, -1), tts_bos], dim=0)        # [L - 1, H]
        rows = self.front(text_ids).float()
        r = c.role_prefix_tokens
        prefill = torch.cat([rows[:r], text_side + codec[:-1], rows[r:r + 1] + codec[-1:]], dim=0)
        trailing = torch.cat([rows[r + 1: len(text_ids) - c.suffix_tokens], tts_eos], dim=0)
        return prefill, trailing, tts_pad

    # ---- sampling ------------------------------------------------------------------------------------------------------
    def _first_code(self, logits: torch.Tensor, seen: torch.Tensor, sp: TTSSampling, step: int) -> int:
        c = self.cfg
        logits = logits.float().clone()
        # control ids never leave the talker, end-of-stream excepted
        eos = logits[:, c.codec_eos_id].clone()
        logits[:, c.codebook_size:] = float("-inf")
        logits[:, c.codec_eos_id] = eos
        if sp.repetition_penalty != 1.0 and seen.any():
            v = logits[:, seen]
            logits[:, seen] = torch.where(v > 0, v / sp.repetition_penalty, v * sp.repetition_penalty)
        params = SamplingParams(temperature=sp.talker_temperature, top_k=sp.talker_top_k, top_p=sp.talker_top_p, seed=sp.seed)
        return int(self.talker.sample(logits, params, step)[0])

    @torch.no_grad()
    def predict_residual_codes(self, talker_hidden: torch.Tensor, first_code: int, sp: TTSSampling, frame: int):
        """The CodePredictor pass of one frame: returns ``(codes 1 … G-1, the sum of their embeddings [1, Ht])``."""
        cp, model = self.predictor, self.predictor.model
        g = self.cfg.num_code_groups
        cp.kv.free(0)
        c0_row = self.talker.embed_tokens([first_code])
        x = model.project(torch.cat([talker_hidden.to(c0_row.dtype), c0_row], dim=0))
        h = cp.prefill_embeds([0], [x])                                       # final-norm hidden of the last row
        params = SamplingParams(temperature=sp.predictor_temperature, top_k=sp.predictor_top_k, top_p=sp.predictor_top_p, seed=sp.seed + 1)
        codes: List[int] = []
        total = torch.zeros_like(c0_row, dtype=torch.float32)
        for j in range(g - 1):
            logits = model.head_logits(h, j)
            code = int(cp.sample(logits, params, frame * g + j)[0])
            codes.append(code)
            row = model.embed(j, torch.tensor([code], device=self.device))
            total += row.float()
            if j + 1 < g - 1:
                h = cp.step_embeds([0], [model.project(row)])
        return codes, total

    @staticmethod
    def _distribution(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
        """The distribution the sampler draws from, as probabilities ``[V]`` (one-hot for greedy settings)."""
        logits = logits.float().reshape(-1)
        if temperature < 1e-3:
            return torch.nn.functional.one_hot(logits.argmax(), logits.numel()).float()
        p = torch.softmax(logits / temperature, dim=-1)
        order = torch.argsort(p, descending=True, stable=True)
        sorted_p = p[order]
        keep = torch.ones_like(sorted_p, dtype=torch.bool)
        if top_k > 0:
            keep[top_k:] = False
        if top_p < 1.0:
            keep &= (sorted_p.cumsum(0) - sorted_p) < top_p
        keep[0] = True
        out = torch.zeros_like(p)
        out[order[keep]] = sorted_p[keep]
        return out / out.sum()

    @torch.no_grad()
    def predict_residual_codes_speculative(self, talker_hidden: torch.Tensor, first_code: int, sp: TTSSampling, frame: int,
                                           generator: Optional[torch.Generator] = None):
        """The CodePredictor pass of one frame with head speculation.  All heads read the same residual stream, so head
        ``j + t`` applied to the hidden state that head ``j`` reads is a draft of the code ``t`` depths ahead at the cost
        of one matrix-vector product.  A round samples the next code from its own head (exact), drafts ``N - 1`` further
        codes from the later heads, feeds all ``N`` embeddings in one pass and checks every draft against the distribution
        its own depth produces: accepted with probability ``min(1, p / q)``, else redrawn from ``max(p - q, 0)`` and the
        round ends there.  The codes are distributed exactly as in the one-code-per-pass loop; with greedy settings they
        are identical.  Returns ``(codes, sum of embeddings, passes)``."""
        cp, model = self.predictor, self.predictor.model
        g, n = self.cfg.num_code_groups, int(sp.cp_spec_verify_size)
        if not 2 <= n <= 8:
            raise ValueError("cp_spec_verify_size must be in 2..8 (one committed depth plus at least one draft)")
        gen = generator or torch.Generator().manual_seed(sp.seed * 7919 + frame)
        dist = lambda lg: self._distribution(lg, sp.predictor_temperature, sp.predictor_top_k, sp.predictor_top_p)   # noqa: E731
        draw = lambda p: int(torch.multinomial(p.cpu(), 1, generator=gen))                                          # noqa: E731
        cp.kv.free(0)
        c0_row = self.talker.embed_tokens([first_code])
        h = cp.prefill_embeds([0], [model.project(torch.cat([talker_hidden.to(c0_row.dtype), c0_row], dim=0))])
        codes: List[int] = []
        total = torch.zeros_like(c0_row, dtype=torch.float32)
        passes = 1

        def commit(code: int) -> torch.Tensor:
            row = model.embed(len(codes), torch.tensor([code], device=self.device))
            codes.append(code)
            total.add_(row.float())
            return row

        while len(codes) < g - 1:
            j = len(codes)                                        # h is the state head j reads
            rows = [commit(draw(dist(model.head_logits(h, j))))]
            if len(codes) == g - 1:
                break
            drafts, q = [], []
            for t in range(1, min(n, g - 1 - j)):
                q.append(dist(model.head_logits(h, j + t)))
                drafts.append(draw(q[-1]))
                rows.append(model.embed(j + t, torch.tensor([drafts[-1]], device=self.device)))
            x = model.project(torch.cat(rows, dim=0))
            meta = cp._meta([0], [x.shape[0]], logits_all=True)
            hs = model(None, meta, cp.cache, inputs_embeds=x.to(model.cfg.compute_dtype))   # one hidden row per fed row
            passes += 1
            accepted = 0
            for t, d in enumerate(drafts):
                p = dist(model.head_logits(hs[t:t + 1], j + 1 + t))
                if float(torch.rand(1, generator=gen)) < min(1.0, float(p[d]) / max(float(q[t][d]), 1e-30)):
                    commit(d)
                    accepted += 1
                    continue
                residual = (p - q[t]).clamp_min(0)
                commit(draw(residual / residual.sum() if float(residual.sum()) > 0 else p))
                break
            # rows kept in the cache: the exact code and the accepted drafts; a redrawn code is fed by the next round
            cp.kv.commit(0, 1 + accepted)
            if accepted == len(drafts):
                h = hs[len(drafts):len(drafts) + 1]
            elif len(codes) < g - 1:
                h = cp.step_embeds([0], [model.project(model.embed(len(codes) - 1, torch.tensor([codes[-1]], device=self.device)))])
                passes += 1
        return codes, total, passes

    # ---- frame loop ----------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_codes(self, text_ids: Sequence[int], speaker: Optional[str] = None, language: Optional[str] = None,
                       sampling: Optional[TTSSampling] = None, on_frames: Optional[Callable[[torch.Tensor, bool], None]] = None,
                       chunk_frames: int = 0):
        """Runs the Talker / CodePredictor loop.  ``on_frames(codes [n, G], is_final)`` is called every ``chunk_frames``
        frames while the loop runs and exactly once with ``is_final`` at the end.  Returns ``(codes [F, G] int32, finish
        reason, talker steps, predictor steps)``."""
        sp = sampling or TTSSampling()
        c = self.cfg
        prefill, trailing, tts_pad = self.build_prefill(text_ids, speaker, language)
        max_frames = min(sp.max_audio_length, self.max_seq_len - prefill.shape[0] - 1)
        if max_frames < 1:
            raise ValueError("the prompt leaves no room for audio frames in the talker's cache")
        tk = self.talker
        tk.kv.free(0)
        logits = tk.prefill_embeds([0], [prefill])
        seen = torch.zeros(logits.shape[-1], dtype=torch.bool, device=logits.device)
        frames: List[List[int]] = []
        sent = 0
        reason = "length"
        talker_steps, predictor_steps = 1, 0
        for f in range(max_frames):
            code0 = self._first_code(logits, seen, sp, f)
            if code0 == c.codec_eos_id:
                reason = "eos"
                break
            seen[code0] = True
            if sp.cp_spec_verify_size:
                rest, rest_sum, passes = self.predict_residual_codes_speculative(tk.model.last_hidden, code0, sp, f)
                predictor_steps += passes
            else:
                rest, rest_sum = self.predict_residual_codes(tk.model.last_hidden, code0, sp, f)
                predictor_steps += c.num_code_groups - 1
            frames.append([code0] + rest)
            if on_frames is not None and chunk_frames > 0 and len(frames) - sent >= chunk_frames:
                on_frames(torch.tensor(frames[sent:], dtype=torch.int32), False)
                sent = len(frames)
            if f + 1 == max_frames:
                break
            nxt = self._codec_rows([code0]) + rest_sum + (trailing[f:f + 1] if f < trailing.shape[0] else tts_pad)
            logits = tk.step_embeds([0], [nxt])
            talker_steps += 1
        codes = torch.tensor(frames, dtype=torch.int32).reshape(-1, c.num_code_groups)
        if on_frames is not None:
            on_frames(codes[sent:], True)
        return codes, reason, talker_steps, predictor_steps

    @torch.no_grad()
    def generate(self, text, speaker: Optional[str] = None, language: Optional[str] = None, sampling: Optional[TTSSampling] = None,
                 chunk_frames: int = 0, on_audio: Optional[Callable[[bytes, int, bool], None]] = None) -> TTSResult:
        """Text (or templated token ids) → audio.  With ``chunk_frames`` the vocoder runs while the loop is still producing
        frames and ``on_audio(pcm16 bytes, sample rate, is_final)`` receives each chunk."""
        ids = self.tokenize(text) if isinstance(text, str) else list(text)
        sr = self.code2wav.cfg.sample_rate
        done: List[torch.Tensor] = []
        pieces: List[torch.Tensor] = []
        chunks = [0]

        def vocode(new: torch.Tensor, final: bool) -> None:
            if new.shape[0]:
                done.append(new)
                all_codes = torch.cat(done, dim=0).t().contiguous().to(self.device)              # [G, F]
                end = all_codes.shape[1]
                wav = self.code2wav.decode_chunk(all_codes, end - new.shape[0], end)
                pieces.append(wav)
                chunks[0] += 1
                if on_audio is not None:
                    on_audio(pcm16_bytes(wav), sr, final)
            elif final and on_audio is not None:
                on_audio(b"", sr, True)

        codes, reason, ts, ps = self.generate_codes(ids, speaker, language, sampling, vocode, chunk_frames)
        wav = torch.cat(pieces) if pieces else torch.zeros(0)
        return TTSResult(codes, wav.float().cpu(), sr, reason, ts, ps, chunks[0])


# ---- artefact directory ------------------------------------------------------------------------------------------------

def _state(module: torch.nn.Module) -> Dict[str, torch.Tensor]:
    return {k: v.detach().cpu().contiguous() for k, v in module.state_dict().items()}


def save_tts(out_dir: str, rt: TTSRuntime) -> str:
    """``tts_config.json`` plus one safetensors file per component (``talker``, ``code_predictor``, ``text``, ``code2wav``)."""
    from safetensors.torch import save_file
    os.makedirs(out_dir, exist_ok=True)
    talker, predictor = rt.talker.model, rt.predictor.model
    meta = {"tts": rt.cfg.to_dict(), "talker": talker.cfg.to_dict(), "code_predictor": predictor.cfg.to_dict(),
            "code2wav": {k: (list(v) if isinstance(v, tuple) else v) for k, v in rt.code2wav.cfg.__dict__.items()},
            "talker_hidden_size": talker.cfg.hidden_size}
    with open(os.path.join(out_dir, TTS_CONFIG_NAME), "w", encoding="utf-8") as f:
        json.dump(meta, f, indent=1)
    for name, mod in (("talker", talker), ("code_predictor", predictor), ("text", rt.front), ("code2wav", rt.code2wav)):
        save_file(_state(mod), os.path.join(out_dir, f"{name}.safetensors"))
    return out_dir


def load_tts(model_dir: str, device="cpu", tokenizer=None, max_seq_len: int = 4096) -> TTSRuntime:
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, TTS_CONFIG_NAME), "r", encoding="utf-8") as f:
        meta = json.load(f)
    cfg = TTSConfig.from_dict(meta["tts"])
    tcfg, pcfg = ModelConfig.from_dict(meta["talker"]), ModelConfig.from_dict(meta["code_predictor"])
    with torch.device(device):
        talker = TalkerCausalLM(tcfg)
        predictor = CodePredictorCausalLM(pcfg, None, cfg.num_code_groups, meta.get("talker_hidden_size", tcfg.hidden_size))
        front = TextFrontEnd(cfg.text_vocab_size, cfg.text_hidden_size, tcfg.hidden_size, tcfg.compute_dtype)
        c2w = Code2Wav(Code2WavConfig.from_dict(meta["code2wav"]))
    for name, mod in (("talker", talker), ("code_predictor", predictor), ("text", front), ("code2wav", c2w)):
        missing, unexpected = mod.load_state_dict(load_file(os.path.join(model_dir, f"{name}.safetensors"), device=str(device)), strict=False)
        if missing or unexpected:
            raise ValueError(f"{name}.safetensors does not match the model: missing {missing[:4]}, unexpected {unexpected[:4]}")
        mod.eval()
        if hasattr(mod, "finalize"):
            mod.finalize()
    if tokenizer is None and os.path.exists(os.path.join(model_dir, "tokenizer.json")):
        from . import native as rt
        tokenizer = rt.Tokenizer(model_dir)
    return TTSRuntime(cfg, talker, predictor, front, c2w, tokenizer, device, max_seq_len)


def random_tts(seed: int = 0, device="cpu", hidden: int = 64, predictor_hidden: int = 32, groups: int = 4, codebook: int = 48,
               text_vocab: int = 96, dtype: str = "float32", max_seq_len: int = 256, head_dim: int = 0) -> TTSRuntime:
    """A small randomly initialised pipeline of the real structure (tests, smoke runs; no checkpoint can be fetched here)."""
    from ..checkpoint.loader import init_random_weights
    ctrl = codebook                                               # control ids follow the audio codes
    cfg = TTSConfig(num_code_groups=groups, codebook_size=codebook, text_vocab_size=text_vocab, text_hidden_size=hidden // 2,
                    codec_pad_id=ctrl, codec_bos_id=ctrl + 1, codec_eos_id=ctrl + 2, codec_think_id=ctrl + 3, codec_nothink_id=ctrl + 4,
                    codec_think_bos_id=ctrl + 5, codec_think_eos_id=ctrl + 6, tts_pad_token_id=text_vocab - 3, tts_bos_token_id=text_vocab - 2,
                    tts_eos_token_id=text_vocab - 1, speakers={"ryan": ctrl + 7, "eric": ctrl + 8}, languages={"english": ctrl + 9, "sichuan_dialect": ctrl + 10},
                    speaker_dialects={"eric": "sichuan_dialect"}, default_speaker="ryan", role_prefix_ids=[1, 2, 3], suffix_ids=[4, 5, 6, 7, 8])
    heads = lambda h: max(2, h // (head_dim or 64))                            # noqa: E731  (head size 64 from hidden 128 up, or as asked)
    tcfg = tiny_llama_config(model_type="qwen3_tts_talker", vocab_size=ctrl + 12, hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=2,
                             num_attention_heads=heads(hidden), num_key_value_heads=heads(hidden) // 2, head_dim=hidden // heads(hidden),
                             has_qk_norm=True, dtype=dtype, max_position_embeddings=max(max_seq_len, 64))
    pcfg = tiny_llama_config(model_type="qwen3_tts_code_predictor", vocab_size=codebook, hidden_size=predictor_hidden,
                             intermediate_size=2 * predictor_hidden, num_hidden_layers=2, num_attention_heads=heads(predictor_hidden),
                             num_key_value_heads=heads(predictor_hidden) // 2, head_dim=predictor_hidden // heads(predictor_hidden),
                             has_qk_norm=True, dtype=dtype, max_position_embeddings=64)
    wcfg = Code2WavConfig(codebook_size=codebook, codebook_dim=16, hidden_size=32, latent_dim=24, num_hidden_layers=2, num_attention_heads=2,
                          intermediate_size=48, sliding_window=4, num_quantizers=groups, upsampling_ratios=(2,), upsample_rates=(3, 2),
                          decoder_dim=32, sample_rate=24000)
    with torch.device(device):
        talker = TalkerCausalLM(tcfg)
        predictor = CodePredictorCausalLM(pcfg, None, groups, hidden)
        front = TextFrontEnd(text_vocab, cfg.text_hidden_size, hidden, tcfg.compute_dtype)
        c2w = Code2Wav(wcfg)
    init_random_weights(talker, seed)
    init_random_weights(predictor, seed + 1)
    g = torch.Generator().manual_seed(seed + 2)
    with torch.no_grad():
        for mod, std in ((predictor, 0.3), (front, 0.3), (c2w, 0.3)):
            for name, p in mod.named_parameters():
                plain = name in ("lm_heads", "codec_embeddings") or name.startswith("small_to_mtp") or mod is not predictor
                if plain and not name.endswith(("layernorm.weight", "norm.weight")) and p.dtype.is_floating_point:
                    p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
    for m in (talker, predictor, front, c2w):
        m.eval()
    return TTSRuntime(cfg, talker, predictor, front, c2w, None, device, max_seq_len)


class TTS:
    """The user-facing class (the reference's Python ``TTS``): ``TTS(model_dir).generate(text, speaker=...)``."""

    def __init__(self, model_dir_or_runtime, device="cpu", **kw):
        self.runtime = model_dir_or_runtime if isinstance(model_dir_or_runtime, TTSRuntime) else load_tts(model_dir_or_runtime, device, **kw)

    def list_voices(self) -> List[str]:
        return self.runtime.voices()

    def generate(self, text, speaker: Optional[str] = None, language: Optional[str] = None, sampling: Optional[TTSSampling] = None,
                 chunk_frames: int = 0, on_audio=None) -> TTSResult:
        return self.runtime.generate(text, speaker, language, sampling, chunk_frames, on_audio)
