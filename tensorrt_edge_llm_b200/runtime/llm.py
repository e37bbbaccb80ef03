"""Offline generation API: ``LLM(...).generate(prompts, SamplingParams)``.

Parity: ``tensorrt_edgellm.server.LLM`` / ``SamplingParams``
(``tensorrt_edgellm/server/runtime/engine.py:920-2167``; usage in
``docs/source/user_guide/examples/server.md:27-64``).  Construction takes a checkpoint directory
or a :class:`ModelConfig` (random-init weights, for benchmarks without network access).
"""
from __future__ import annotations

import dataclasses
import os
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Union

import torch

from ..config import (QUANT_NVFP4, Mapping, ModelConfig, QuantConfig)
from ..model import AutoModel
from .kv_cache import KVCacheManager
from . import logits as lp
from .runner import ModelRunner, SamplingParams


@dataclass
class RequestOutput:
    prompt_token_ids: List[int]
    token_ids: List[int]
    text: Optional[str] = None
    finish_reason: str = "length"
    ttft_s: float = 0.0
    decode_s: float = 0.0
    logprobs: Optional[List[dict]] = None      # per token: {"token_id", "logprob", "top": [(id, logprob), ...]}
    reused_input_tokens: int = 0               # prompt tokens served from the prefix cache
    spec_stats: Optional[dict] = None          # speculative runs: rounds, draft forwards, mean acceptance length


def ifb_unsupported_reason(*, speculative: bool = False, reduced_vocab: bool = False, debug_hooks: bool = False) -> Optional[str]:
    """Why a deployment cannot use the in-flight-batching engine, or ``None`` (``ifb_unsupported_reason`` of the
    reference's ``server/runtime/engine.py``).  The debug hooks (layer dumps, forced tokens) run on the static-batch path
    only; speculative decoding is scheduled by the engine (one draft → verify round per step and resident row)."""
    if speculative and reduced_vocab:
        return "speculative decoding verifies over the full vocabulary"
    if debug_hooks:
        return "layer dumps / forced tokens need the static-batch path"
    return None


class LLM:
    def __init__(self, model: Union[str, ModelConfig], *, device: Optional[str] = None, comm=None,
                 max_batch_size: int = 64, max_input_len: int = 2048, max_kv_cache_capacity: int = 2304,
                 page_size: int = 64, max_num_tokens: int = 8192, random_init_seed: Optional[int] = 0,
                 tokenizer=None, kv_pages: Optional[int] = None, enable_in_flight_batching: bool = False,
                 enable_prefix_cache: bool = False, scheduling: Optional[dict] = None, draft_model=None, speculative=None,
                 context_cache_max_records: int = 4096, context_cache_max_snapshots: int = 64,
                 embedding_quantization: Optional[str] = None, tp_mirror=None, mapping: Optional[Mapping] = None,
                 kv_cache_dtype: Optional[str] = None):
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if isinstance(model, ModelConfig):
            self.model = AutoModel.from_config(model, comm=comm, device=self.device, random_init=random_init_seed)
        else:
            self.model = AutoModel.from_pretrained(model, comm=comm, device=self.device, **({"mapping": mapping} if mapping else {}))
        self.cfg = self.model.cfg
        if embedding_quantization:                  # "fp8" | "nvfp4": the token table is stored quantised, rows expand on lookup
            from ..models.embedding import quantize_embedding
            quantize_embedding(self.model, embedding_quantization)
        self.tokenizer = tokenizer
        self._vocab_map = None
        if isinstance(model, str):
            self._vocab_map = self._load_reduced_vocab(model)
        self.max_batch_size = max_batch_size
        self.max_input_len = max_input_len
        # block-diffusion checkpoints write a whole canvas beyond the committed tokens in every denoise pass
        canvas_headroom = self.cfg.diffusion.canvas_length if self.cfg.diffusion is not None else 0
        pages_per_seq = (max_kv_cache_capacity + canvas_headroom + page_size - 1) // page_size
        total_pages = kv_pages or (pages_per_seq * max_batch_size + 1)
        # "fp8": E4M3 KV pages (`--kv-cache-quantization fp8` checkpoints select it through their quantisation config)
        self.kv = KVCacheManager(self.cfg, total_pages, page_size, max_seats=max_batch_size,
                                 max_pages_per_seq=pages_per_seq, device=self.device, kv_dtype=kv_cache_dtype)
        self.runner = ModelRunner(self.model, self.kv, self.device, max_num_tokens=max_num_tokens)
        self.runner.vocab_map = self._vocab_map
        self.lora = None
        self.runner.lora = None
        slots = os.path.join(model, "lora_slots.json") if isinstance(model, str) else ""
        if slots and os.path.isfile(slots):         # adapter slots declared ahead of time (`trtedge insert-lora --model_dir`)
            from ..lora.runtime import LoraManager
            self.lora = LoraManager(self.model)
            self.runner.lora = self.lora
            self.lora.reserve_slots(slots)
        eos0 = self.cfg.eos_token_id
        self.guided_vocab = lp.GuidedVocabulary(tokenizer, self.cfg.vocab_size, eos0 if isinstance(eos0, (list, tuple)) else [eos0])
        self.engine = None
        # Speculative decoding (EAGLE-3 / MTP draft head): greedy requests on the static-batch path run draft → verify rounds.
        self.spec_decoder = None
        self.diffusion_decoder = None
        if self.cfg.diffusion is not None:
            if draft_model is not None or enable_in_flight_batching:
                raise ValueError("block-diffusion checkpoints decode whole blocks: no draft model, no in-flight batching")
            from .block_diffusion import BlockDiffusionDecoder
            self.diffusion_decoder = BlockDiffusionDecoder(self.runner)
        if draft_model is not None:
            from .speculative import EagleDecoder, SpecConfig
            draft = (AutoModel.from_config(draft_model, device=self.device, random_init=random_init_seed)
                     if isinstance(draft_model, ModelConfig) else AutoModel.from_pretrained(draft_model, device=self.device))
            if hasattr(draft, "share_lm_head") and not isinstance(draft_model, ModelConfig):
                draft.share_lm_head(self.model)
            spec = speculative or SpecConfig()
            is_dflash = draft.cfg.draft_type == "dflash"
            block_tree = is_dflash and spec.block_tree_top_k > 1 and not hasattr(draft, "propose_tokens")
            headroom = (max(draft.cfg.dflash_block_size, min(spec.verify_tokens, 64) if block_tree else 0) + 8 if is_dflash
                        else spec.verify_tokens + spec.draft_steps * spec.top_k)
            sp_pages = (max_kv_cache_capacity + headroom + page_size - 1) // page_size
            self.kv = KVCacheManager(self.cfg, (kv_pages or sp_pages * max_batch_size + 1), page_size, max_seats=max_batch_size,
                                     max_pages_per_seq=sp_pages, device=self.device, kv_dtype=kv_cache_dtype)
            self.runner = ModelRunner(self.model, self.kv, self.device, max_num_tokens=max_num_tokens)
            dkv = KVCacheManager(draft.cfg, sp_pages * max_batch_size + 1, page_size, max_seats=max_batch_size, max_pages_per_seq=sp_pages,
                                 device=self.device, num_layers=draft.cfg.num_hidden_layers if is_dflash else 1)
            if is_dflash:                      # block draft over target-derived keys / values (runtime/dflash.py)
                from .dflash import DFlashDecoder
                self.spec_decoder = DFlashDecoder(self.runner, draft, dkv, tree_top_k=spec.block_tree_top_k if block_tree else 1,
                                                  verify_tokens=min(spec.verify_tokens, 64) if block_tree else 0)
            else:
                self.spec_decoder = EagleDecoder(self.runner, draft, dkv, spec)
        from .debug import LayerDumper, forced_tokens_from_env
        self._dumper = LayerDumper.from_env()
        if self._dumper is not None:
            self._dumper.attach(self.model)
            self.runner.use_cuda_graphs = False        # hooks do not run inside a replayed graph
        self._forced = forced_tokens_from_env()
        self._tp_mirror = tp_mirror
        if enable_in_flight_batching:
            if self.cfg.tp_size > 1 and tp_mirror is None:
                raise ValueError("in-flight batching with tensor parallelism needs tp_mirror (rank 0 schedules, the other ranks run "
                                 "parallel.tp_serving.serve_follower)")
            why = ifb_unsupported_reason(debug_hooks=self._dumper is not None or self._forced is not None)
            if why:
                raise ValueError(f"in-flight batching cannot be enabled: {why}")
            self._cache_limits = (int(context_cache_max_records), int(context_cache_max_snapshots) or 64)
            self._start_engine(enable_prefix_cache, scheduling or {})

    # ---- LoRA adapters ------------------------------------------------------------------------------
    def load_lora(self, name: str, adapter_dir: str) -> None:
        """Load a processed adapter (``trtedge process-lora``) under ``name``; requests choose it with
        ``SamplingParams(lora_name=...)`` (``cpp/runtime/state/loraManager`` in the reference: named adapters, switched per
        request without touching the base weights)."""
        if self.lora is None:
            from ..lora.runtime import LoraManager
            self.lora = LoraManager(self.model)
            self.runner.lora = self.lora
        self.lora.load_adapter(name, adapter_dir)

    def _load_reduced_vocab(self, model_dir: str):
        """``vocab_map.safetensors`` next to the checkpoint (``trtedge reduce-vocab``): swap in the reduced LM head."""
        import os
        from ..checkpoint.safetensors_io import SafetensorsFile
        p = os.path.join(model_dir, "vocab_map.safetensors")
        if not os.path.exists(p) or self.cfg.tp_size > 1:
            return None
        f = SafetensorsFile(p)
        from ..models.linear import Linear
        w = f.get("lm_head.weight")
        dtype = next(self.model.parameters()).dtype
        head = Linear(w.shape[1], [w.shape[0]], dtype=dtype)
        head.weight.data.copy_(w.to(dtype))
        self.model.lm_head = head.to(self.device)
        return f.get("vocab_map").clone().to(self.device, torch.int32)

    # ---- in-flight batching --------------------------------------------------------------------------
    def _start_engine(self, enable_prefix_cache: bool, scheduling: dict) -> None:
        """Start the native request engine (actor thread) over a model session."""
        from . import native as rt
        from .session import ModelSession
        eos = self.cfg.eos_token_id
        eos_ids = eos if isinstance(eos, (list, tuple)) else [eos]
        cfg = rt.EngineConfig()
        cfg.max_batch_size = self.max_batch_size
        opts = rt.SchedulingOptions()
        if self.spec_decoder is not None:
            # the draft must see whole prompts: no chunked prefill, and a step budget that holds the longest prompt
            scheduling = {**scheduling, "max_chunk_tokens": self.max_input_len,
                          "max_num_tokens": max(int(scheduling.get("max_num_tokens", 0) or 0), self.max_input_len + self.max_batch_size)}
        for k, v in scheduling.items():
            if k == "mode":
                v = {"auto": rt.IfbSchedulingMode.Auto, "mixed": rt.IfbSchedulingMode.Mixed,
                     "prefill_first": rt.IfbSchedulingMode.PrefillFirst, "single_cohort": rt.IfbSchedulingMode.SingleCohort}[v]
            elif k == "policy":
                v = {"fcfs": rt.SchedulingPolicy.Fcfs, "priority": rt.SchedulingPolicy.Priority}[v]
            elif k == "preemption":
                v = {"none": rt.PreemptionMode.NoPreemption, "pause": rt.PreemptionMode.Pause}[v]
            setattr(opts, k, v)
        cfg.scheduling = opts
        self._rt = rt
        def make_session():
            self.session = ModelSession(self.runner, eos_ids, enable_prefix_cache, self.max_input_len, self.guided_vocab,
                                        max_snapshots=self._cache_limits[1], max_records=self._cache_limits[0],
                                        spec_decoder=self.spec_decoder, mirror=self._tp_mirror)
            return self.session             # kept for its counters (prefix hits, jump-forward tokens); the engine thread owns it
        # With a native tokenizer the engine sits inside the native façade (csrc/runtime/inference_runtime.cpp), which adds
        # handle_request (chat rendering, tokenisation, incremental detokenisation, textual stop sequences) on top of the same
        # submit / metrics / status surface; otherwise the bare request engine.
        self.native_runtime = None
        if isinstance(self.tokenizer, rt.Tokenizer):
            self.native_runtime = rt.LLMInferenceRuntime(cfg, make_session, self.tokenizer, getattr(self, "native_chat_template", None),
                                                         self.spec_decoder is not None, None)
            self.engine = self.native_runtime
        else:
            self.engine = rt.RequestEngine(cfg, make_session)

    def _native_request(self, ids, sp: SamplingParams, priority: int = 0):
        r = self._rt.GenerationRequest()
        r.prompt_ids = [int(t) for t in ids]
        r.max_tokens, r.temperature, r.top_k, r.top_p = sp.max_tokens, sp.temperature, sp.top_k, sp.top_p
        r.seed, r.ignore_eos, r.stop_token_ids, r.priority = sp.seed, sp.ignore_eos, list(sp.stop_token_ids), priority
        if sp.logprobs is not None:
            r.num_logprobs = int(sp.logprobs)
        if sp.logit_bias:
            r.logit_bias_ids = [int(k) for k in sp.logit_bias]
            r.logit_bias_values = [float(v) for v in sp.logit_bias.values()]
        if sp.guided is not None:
            r.guided_type, r.guided_spec = lp.guided_to_wire(sp.guided)
        if sp.lora_name:
            if self.lora is None or sp.lora_name not in self.lora.names:
                raise ValueError(f"unknown LoRA adapter {sp.lora_name!r}")
            r.lora_name = sp.lora_name
        r.disable_spec_decode = bool(sp.disable_spec_decode)
        r.cache_lookup = bool(sp.context_cache_lookup)
        try:
            r.cache_commit = {"none": 0, "prefill_state_only": 1, "including_generated_tokens": 2}[sp.context_cache_commit]
        except KeyError:
            raise ValueError(f"unknown context_cache_commit policy {sp.context_cache_commit!r}") from None
        return r

    @staticmethod
    def _logprob_rows(tokens, rep) -> Optional[List[dict]]:
        """Native ``TokenLogprobs`` → one dict per generated token."""
        if rep is None or not rep.chosen:
            return None
        n = len(rep.chosen)
        k = len(rep.top_ids) // n if n else 0
        return [{"token_id": int(tokens[i]) if i < len(tokens) else None, "logprob": float(rep.chosen[i]),
                 "top": [(int(rep.top_ids[i * k + j]), float(rep.top_values[i * k + j])) for j in range(k)]} for i in range(n)]

    def submit(self, prompt, sampling_params: Optional[SamplingParams] = None, priority: int = 0):
        """Queue one request on the in-flight-batching engine; returns the native ``RequestHandle``
        (``.get()``, ``.stream()``, ``.cancel()``, ``.stats()``).  Raises when the engine refuses it."""
        if self.engine is None:
            raise RuntimeError("LLM was built without enable_in_flight_batching")
        ids = self._encode([prompt])[0]
        if hasattr(ids, "embeds"):
            return self.submit_multimodal(ids.ids, ids.embeds, sampling_params, ids.positions3, ids.rope_delta, ids.deepstack, priority)
        h, why = self.engine.submit(self._native_request(ids, sampling_params or SamplingParams(), priority))
        if h is None:
            raise RuntimeError(why)
        return h

    # ---- counters (the names of the reference's Python runtime) ------------------------------------------
    def get_scheduling_metrics(self) -> Optional[dict]:
        """Counters of the request engine (``None`` without in-flight batching): submissions, completions, step kinds,
        mid-flight admissions, stalls — ``cpp/scheduler/requestEngine.cpp:507-563`` in the reference."""
        if self.engine is None:
            return None
        m = self.engine.metrics()
        names = ("submitted", "refused", "completed", "cancelled", "failed", "admitted_mid_flight", "stalls_no_capacity", "stalls_exclusive",
                 "decode_steps", "prompt_steps", "mixed_steps", "step_tokens", "paused_resident_steps", "session_failures")
        return {**{k: int(getattr(m, k)) for k in names}, "queue_latency_s_sum": float(m.queue_latency_s_sum)}

    def list_voices(self) -> List[str]:
        """Voices of a speech synthesis stage (the reference's ``LLM.list_voices``); this runtime loads none."""
        return []

    def get_context_cache_counters(self) -> Optional[dict]:
        """Prefix-reuse counters (``None`` when context reuse is off)."""
        sess = getattr(self, "session", None)
        if self.engine is None or sess is None or sess.prefix is None:
            return None
        return {"reused_tokens": int(self.engine.metrics().prefix_reused_tokens), "snapshot_hits": int(sess.snapshot_hits),
                "snapshots": len(sess.snapshots), "jump_forward_tokens": int(sess.jump_forward_tokens)}

    def submit_multimodal(self, ids: Sequence[int], embeds: torch.Tensor, sampling_params: Optional[SamplingParams] = None, positions3=None,
                          rope_delta: int = 0, deepstack: Optional[dict] = None, priority: int = 0):
        """Queue a multimodal prompt on the request engine: ``ids`` hold placeholder tokens where media sits, ``embeds`` the
        rows actually fed (``runtime.multimodal.MultimodalRunner.build`` makes both).  Returns the request handle."""
        if self.engine is None:
            raise RuntimeError("submit_multimodal needs in-flight batching")
        sp = sampling_params or SamplingParams()
        req = self._native_request([int(t) for t in ids], sp, priority)
        req.embeds_key = self.session.register_embeds(list(ids), embeds, positions3, rope_delta, deepstack)
        req.cache_lookup = False
        h, why = self.engine.submit(req)
        if h is None:
            self.session.mm_store.pop(int(req.embeds_key), None)
            raise RuntimeError(why)
        return h

    def generate_stream(self, prompt, sampling_params: Optional[SamplingParams] = None, on_metrics=None):
        """Yield ``(token_ids, text_delta)`` chunks as they are produced."""
        h = self.submit(prompt, sampling_params)
        ch = h.stream()
        pending = b""
        while True:
            c = ch.wait_pop(1.0)
            if c is None:
                continue
            text = None
            if self.tokenizer is not None and hasattr(self.tokenizer, "id_to_bytes"):
                for t in c.token_ids:
                    pending += bytes(self.tokenizer.id_to_bytes(t))
                n = self._rt.utf8_complete_prefix(pending)        # never emit half a UTF-8 character
                text, pending = pending[:n].decode("utf-8", "replace"), pending[n:]
            if c.token_ids or c.finished:
                yield c.token_ids, text
            if c.finished:
                break
        if on_metrics is not None:
            on_metrics(ch.metrics())

    # ------------------------------------------------------------------------------------------
    def _encode(self, prompts) -> List[List[int]]:
        out = []
        for p in prompts:
            if hasattr(p, "embeds") and hasattr(p, "ids"):        # runtime.multimodal.MultimodalPrompt: passes through as it is
                out.append(p)
            elif isinstance(p, str):
                if self.tokenizer is None:
                    raise ValueError("text prompts need a tokenizer")
                out.append(list(self.tokenizer.encode(p)))
            else:
                out.append([int(t) for t in p])
        return out

    @torch.no_grad()
    def generate(self, prompts: Sequence[Union[str, Sequence[int]]], sampling_params: Optional[SamplingParams] = None
                 ) -> List[RequestOutput]:
        """Generate for a batch of prompts (static batch: one prefill wave, then decode)."""
        sp = sampling_params or SamplingParams()
        if os.environ.get("EDGELLM_IGNORE_EOS", "0") == "1" and not sp.ignore_eos:      # benchmark switch of the reference
            sp = dataclasses.replace(sp, ignore_eos=True)
        if self.engine is not None:
            if isinstance(prompts, torch.Tensor):
                prompts = prompts.tolist()
            ids = self._encode(prompts)
            handles = [self.submit(p, sp) for p in ids]
            outs = []
            for p, h in zip(ids, handles):
                toks = h.get(3600.0)
                st = h.stats()
                reason = {self._rt.FinishReason.Length: "length", self._rt.FinishReason.EndId: "stop",
                          self._rt.FinishReason.StopWords: "stop", self._rt.FinishReason.Cancelled: "cancelled",
                          self._rt.FinishReason.Error: "error"}.get(h.reason(), "length")
                text = self.tokenizer.decode(toks) if self.tokenizer is not None else None
                if reason == "error" and h.error():
                    raise ValueError(h.error()) if "EDGELLM_BAD_REQUEST" in h.error() else RuntimeError(h.error())
                outs.append(RequestOutput(list(p), toks, text, reason, st.ttft_s, max(st.total_s - st.ttft_s, 0.0),
                                          self._logprob_rows(toks, h.logprobs()), int(st.reused_tokens)))
            return outs
        if isinstance(prompts, torch.Tensor):
            outs = []
            for b0 in range(0, prompts.shape[0], self.max_batch_size):
                outs.extend(self._generate_batch(prompts[b0:b0 + self.max_batch_size], sp))
            return outs
        ids = self._encode(prompts)
        outs: List[RequestOutput] = []
        if any(hasattr(p, "embeds") for p in ids):        # prepared multimodal prompts: one at a time on the static path
            for p in ids:
                outs.extend([self._generate_multimodal_static(p, sp)] if hasattr(p, "embeds") else self._generate_batch([p], sp))
            return outs
        for b0 in range(0, len(ids), self.max_batch_size):
            outs.extend(self._generate_batch(ids[b0:b0 + self.max_batch_size], sp))
        return outs

    def _generate_multimodal_static(self, p, sp: SamplingParams) -> RequestOutput:
        """A prepared multimodal prompt without the request engine: prefill from its embedding rows, then ordinary decode."""
        if sp.needs_logits_processing:
            raise ValueError("constrained / biased decoding of multimodal prompts needs in-flight batching")
        seat, runner = 0, self.runner
        self.kv.free(seat)
        self.kv.reserve(seat, len(p) + sp.max_tokens)
        t0 = time.perf_counter()
        pos3 = None if p.positions3 is None else [p.positions3]
        logits = runner.prefill_embeds([seat], [p.embeds], positions3=pos3, rope_deltas=None if pos3 is None else [p.rope_delta],
                                       deepstack=p.deepstack)
        first = runner.sample(logits, sp, step=0)
        t1 = time.perf_counter()
        toks = [int(first[0])]
        if sp.max_tokens > 1:
            rest = (runner.decode_greedy([seat], first, sp.max_tokens - 1) if sp.temperature < 1e-3
                    else runner.decode_sampled([seat], first, sp.max_tokens - 1, sp))
            toks += rest[0].tolist()
        self.kv.free(seat)
        eos = self.cfg.eos_token_id
        eos_set = (set(eos if isinstance(eos, (list, tuple)) else [eos]) - {None}) | set(sp.stop_token_ids)
        reason = "length"
        if not sp.ignore_eos:
            for j, t in enumerate(toks):
                if t in eos_set:
                    toks, reason = toks[:j + 1], "stop"
                    break
        text = self.tokenizer.decode(toks) if self.tokenizer is not None else None
        return RequestOutput(list(p.ids), toks, text, reason, t1 - t0, time.perf_counter() - t1)

    def _generate_diffusion(self, ids: List[List[int]], sp: SamplingParams) -> List[RequestOutput]:
        """Block-diffusion checkpoints: denoise and commit one canvas at a time (``runtime/block_diffusion.py``).  The
        model's own sampler replaces temperature / top-k / top-p; ``seed`` seeds the canvas and Gumbel noise."""
        if sp.needs_logits_processing:
            raise ValueError("block-diffusion decoding takes no logit bias, log-probabilities or output constraints")
        dec = self.diffusion_decoder
        for p in ids:
            if len(p) > self.max_input_len:
                raise ValueError(f"prompt of {len(p)} tokens exceeds max_input_len {self.max_input_len}")
        eos = self.cfg.eos_token_id
        eos_set = set(eos if isinstance(eos, (list, tuple)) else [eos]) if eos is not None else set()
        eos_set |= set(sp.stop_token_ids)
        seats = list(range(len(ids)))
        b0, p0 = dec.stats.blocks, dec.stats.denoise_passes
        t0 = time.perf_counter()
        toks = dec.generate(seats, ids, sp.max_tokens, () if sp.ignore_eos else sorted(eos_set),
                            max_denoising_steps=int(sp.max_denoising_steps or 0), seed=sp.seed)
        t1 = time.perf_counter()
        stats = {"blocks": dec.stats.blocks - b0, "denoise_passes": dec.stats.denoise_passes - p0}
        outs = []
        for p, row in zip(ids, toks):
            reason = "stop" if (row and not sp.ignore_eos and row[-1] in eos_set) else "length"
            text = self.tokenizer.decode(row) if self.tokenizer is not None else None
            outs.append(RequestOutput(list(p), row, text, reason, 0.0, t1 - t0, spec_stats=stats))
        for s in seats:
            self.kv.free(s)
        return outs

    def _generate_speculative(self, ids: List[List[int]], sp: SamplingParams) -> List[RequestOutput]:
        """Greedy generation through draft → tree verify rounds (lossless: same tokens as plain greedy decoding)."""
        dec = self.spec_decoder
        n = len(ids)
        seats = list(range(n))
        dec.release(seats)
        eos = self.cfg.eos_token_id
        eos_id = None if sp.ignore_eos else (eos[0] if isinstance(eos, (list, tuple)) and eos else eos)
        r0, e0, d0 = dec.stats.rounds, dec.stats.emitted, dec.stats.draft_forwards
        t0 = time.perf_counter()
        sampling = None if sp.temperature < 1e-3 else {"temperature": sp.temperature, "top_k": sp.top_k, "top_p": sp.top_p, "seed": sp.seed}
        toks = dec.generate(seats, [list(map(int, p)) for p in ids], sp.max_tokens, eos_id, sampling=sampling)
        t1 = time.perf_counter()
        rounds = dec.stats.rounds - r0
        stats = {"verify_rounds": rounds, "draft_forwards": dec.stats.draft_forwards - d0,
                 "mean_acceptance_length": (dec.stats.emitted - e0) / max(rounds, 1)}
        dec.release(seats)
        outs = []
        for p, row in zip(ids, toks):
            reason = "stop" if (eos_id is not None and row and row[-1] == eos_id) else "length"
            text = self.tokenizer.decode(row) if self.tokenizer is not None else None
            outs.append(RequestOutput(list(p), row, text, reason, 0.0, t1 - t0, spec_stats=stats))
        return outs

    def _generate_processed(self, ids: List[List[int]], sp: SamplingParams) -> List[RequestOutput]:
        """Static-batch generation with per-step logits processing (bias, constraint mask, log-probabilities)."""
        n = len(ids)
        seats = list(range(n))
        for s in seats:
            self.kv.free(s)
        for s, p in zip(seats, ids):
            self.kv.reserve(s, len(p) + sp.max_tokens)
        states = [lp.make_row_state(self.guided_vocab, guided=sp.guided, logit_bias=sp.logit_bias, num_logprobs=sp.logprobs,
                                    vocab_size=self.cfg.vocab_size) for _ in range(n)]
        eos = self.cfg.eos_token_id
        eos_set = set(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]) if e is not None) | set(sp.stop_token_ids)
        was, self.runner.use_cuda_graphs = self.runner.use_cuda_graphs, False
        rows: List[List[int]] = [[] for _ in range(n)]
        reports: List[List[dict]] = [[] for _ in range(n)]
        reasons = ["length"] * n
        live = list(range(n))
        feed: List[List[int]] = [[] for _ in range(n)]
        self.jump_forward_tokens = 0
        t0 = time.perf_counter()
        try:
            logits = self.runner.prefill(seats, [list(map(int, p)) for p in ids])
            t1 = time.perf_counter()
            for step in range(sp.max_tokens):
                st = [states[i] for i in live]
                proc = lp.process(logits, st)
                toks = [int(t) for t in self.runner.sample(proc, sp, step=step).tolist()]
                reps = lp.logprobs(proc, toks, st)
                done = lp.advance(st, toks)
                keep = []
                for j, i in enumerate(live):
                    if done[j]:
                        reasons[i] = "stop"
                        continue
                    rows[i].append(toks[j])
                    if reps[j] is not None:
                        reports[i].append({"token_id": toks[j], "logprob": reps[j].chosen[0],
                                           "top": list(zip(reps[j].top_ids[0], reps[j].top_values[0]))})
                    if not sp.ignore_eos and toks[j] in eos_set:
                        reasons[i] = "stop"
                        continue
                    feed[i] = [toks[j]]
                    dec = states[i].guided
                    if dec is not None and dec.jump_forward:          # grammar-forced tokens ride along with the sampled one
                        extra = dec.forced_tokens(self.tokenizer, sp.max_tokens - len(rows[i]))
                        rows[i] += extra
                        feed[i] += extra
                        self.jump_forward_tokens += len(extra)
                    if len(rows[i]) >= sp.max_tokens:
                        continue
                    keep.append(j)
                if not keep:
                    break
                live_next = [live[j] for j in keep]
                logits = self.runner.step([seats[i] for i in live_next], [feed[i] for i in live_next])
                live = live_next
        finally:
            self.runner.use_cuda_graphs = was
            for s in seats:
                self.kv.free(s)
        t2 = time.perf_counter()
        return [RequestOutput(list(ids[i]), rows[i], self.tokenizer.decode(rows[i]) if self.tokenizer is not None else None, reasons[i],
                              t1 - t0, t2 - t1, reports[i] or None) for i in range(n)]

    def _generate_batch(self, ids: List[List[int]], sp: SamplingParams) -> List[RequestOutput]:
        if self.lora is not None:                      # static batch: one adapter (or none) for every row
            if sp.lora_name and sp.lora_name not in self.lora.names:
                raise ValueError(f"unknown LoRA adapter {sp.lora_name!r}")
            self.lora.set_segments(None)
            self.lora.set_active(sp.lora_name)
        if self.diffusion_decoder is not None:
            return self._generate_diffusion([p.tolist() for p in ids] if isinstance(ids, torch.Tensor) else ids, sp)
        if sp.needs_logits_processing:
            return self._generate_processed([p.tolist() for p in ids] if isinstance(ids, torch.Tensor) else ids, sp)
        greedy_only = self.cfg.is_hybrid
        if self.spec_decoder is not None and not isinstance(ids, torch.Tensor) and (sp.temperature < 1e-3 or not greedy_only):
            return self._generate_speculative(ids, sp)
        n = len(ids)
        seats = list(range(n))
        for s in seats:
            self.kv.free(s)
        for s, p in zip(seats, ids):
            if len(p) > self.max_input_len:
                raise ValueError(f"prompt of {len(p)} tokens exceeds max_input_len {self.max_input_len}")
            self.kv.reserve(s, len(p) + sp.max_tokens)
        t0 = time.perf_counter()
        if isinstance(ids, torch.Tensor):
            logits = self.runner.prefill_tensor(seats, ids)      # pinned host tensor → one H2D copy per chunk
        else:
            logits = self.runner.prefill(seats, ids)
        first = self.runner.sample(logits, sp, step=0)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t1 = time.perf_counter()
        if self._forced is not None:
            # teacher forcing: feed the listed ids step by step and return them as the output
            forced = [self._forced[i][:sp.max_tokens] for i in range(n)]
            for k in range(max(len(f) for f in forced) - 1):
                self.runner.step(seats, [[f[min(k, len(f) - 1)]] for f in forced])
            toks = torch.tensor([f + [f[-1]] * (sp.max_tokens - len(f)) for f in forced], dtype=torch.int32)
        elif sp.max_tokens > 1:
            if sp.temperature < 1e-3:
                rest = self.runner.decode_greedy(seats, first, sp.max_tokens - 1)
            else:
                rest = self.runner.decode_sampled(seats, first, sp.max_tokens - 1, sp)
            toks = torch.cat([first[:, None].to(rest.device), rest], dim=1)
        else:
            toks = first[:, None]
        toks_host = toks.to("cpu")          # device → host read of the step's result
        t2 = time.perf_counter()
        outs = []
        eos = self.cfg.eos_token_id
        eos_set = set(eos if isinstance(eos, (list, tuple)) else [eos]) if eos is not None else set()
        eos_set |= set(sp.stop_token_ids)
        for i in range(n):
            row = toks_host[i].tolist()
            reason = "length"
            if not sp.ignore_eos and eos_set:
                for j, t in enumerate(row):
                    if t in eos_set:
                        row = row[:j + 1]
                        reason = "stop"
                        break
            text = self.tokenizer.decode(row) if self.tokenizer is not None else None
            outs.append(RequestOutput(ids[i].tolist() if isinstance(ids, torch.Tensor) else ids[i], row, text, reason,
                                      t1 - t0, t2 - t1))
        for s in seats:
            self.kv.free(s)
        return outs

    def refit(self, source, names=None, timeout_s: float = 60.0) -> dict:
        """Replace weights of the live model in place (``checkpoint/external_weights.py: refit``): ``source`` is a safetensors
        file or a ``name → tensor`` dict named as the model's state (an artefact directory's ``rank<r>.external.safetensors``,
        for instance).  Waits for the request engine to drain first; cached K/V of the old weights is never reused afterwards
        (a new prefix-cache generation).  Tensor addresses do not change, so captured graphs stay valid."""
        import time
        from ..checkpoint.external_weights import refit as _refit
        if self.engine is not None:
            t0 = time.monotonic()
            while self.engine.queued() or self.engine.resident():
                if time.monotonic() - t0 > timeout_s:
                    raise TimeoutError("refit: the request engine did not drain in time")
                time.sleep(0.005)
        stats = _refit(self.model, source, names)
        self.runner.weights_epoch = int(getattr(self.runner, "weights_epoch", 0)) + 1
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        return stats

    def close(self):
        if self.engine is not None:
            self.engine.shutdown()
            self.engine = None
            if self._tp_mirror is not None:
                self._tp_mirror.send(("stop",))
        self.runner = None
        self.kv = None
        self.model = None
