"""The runtime objects under the names of the reference's Python runtime module.

The reference binds its C++ runtime with nanobind (``python/nanobind/bindings.cpp``: ``LLMRuntime`` :1359-1371,
``StreamChannel`` :1484-1509, ``RequestHandle`` / ``RequestEngine`` :1649-1706, ``MultiStageRuntime`` :1781-1821,
``validate_scheduling_options``) and re-exports the classes from ``tensorrt_edgellm.runtime``.  Here the scheduler side
(``RequestEngine``, ``RequestHandle``, ``StreamChannel``, scheduling options, planner, sessions) *is* native code — the
pybind11 module ``_telb_runtime`` — and is re-exported unchanged; ``LLMRuntime`` is the request-file façade of
``cpp/runtime/llmInferenceRuntime.h:59-156`` (``handleRequest``, ``countPromptTokens``, ``captureDecodingCUDAGraph``,
``openSession`` …) over this package's ``LLM`` object, whose "engine" is the module of sm_100a kernels rather than a
TensorRT plan file.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

from .llm import LLM
from .runner import SamplingParams


class LLMRuntime:
    """One loaded model that answers request files (``docs/source/user_guide/format/input-format.md``).

    ``LLMRuntime(engine_dir)`` loads a checkpoint directory (there is no engine build step); keyword arguments are those of
    :class:`LLM`.  ``handle_request`` takes the parsed request file (a dict, or its JSON text) and returns the response dict
    of ``examples/cpp/llm_inference`` (``responses[].output_text`` …); the batch is decoded together when the file's
    ``batch_size`` allows it."""

    def __init__(self, engine_dir, multimodal_engine_dir: Optional[str] = None, lora_weights: Optional[Dict[str, str]] = None,
                 llm: Optional[LLM] = None, **llm_kwargs):
        from ..chat_template import ChatTemplate
        if llm is None:
            tokenizer = llm_kwargs.pop("tokenizer", None)
            if tokenizer is None and isinstance(engine_dir, str) and os.path.exists(os.path.join(engine_dir, "tokenizer.json")):
                from . import native as rt
                tokenizer = rt.Tokenizer.load_from_hf(engine_dir)
            llm = LLM(engine_dir, tokenizer=tokenizer, **llm_kwargs)
        self.llm = llm
        self.template = ChatTemplate.load(engine_dir) if isinstance(engine_dir, str) and hasattr(ChatTemplate, "load") else ChatTemplate()
        for name, path in (lora_weights or {}).items():
            self.llm.load_lora(name, path)
        self._unavailable = ""
        self._last: Dict[str, Any] = {}

    # ---- llmInferenceRuntime.h surface ---------------------------------------------------------------------
    def handle_request(self, request) -> Dict[str, Any]:
        """Run every request of a request file; returns ``{"responses": [...]}`` (``LLMGenerationResponse``: output ids and
        text, finish reason, token counts, optional log-probabilities and speculative-decoding statistics)."""
        from ..commands.infer import parse_request_file, run_requests
        body = json.loads(request) if isinstance(request, (str, bytes)) else request
        try:
            parsed = parse_request_file(body)
            responses = run_requests(self.llm, self.template, parsed)
        except RuntimeError as e:              # a device-side failure makes the runtime unusable until it is rebuilt
            self._unavailable = str(e)
            raise
        self._last = {"requests": len(parsed), "output_tokens": sum(r["output_tokens"] for r in responses),
                      "input_tokens": sum(r["input_tokens"] for r in responses)}
        return {"responses": responses}

    def count_prompt_tokens(self, request) -> List[int]:
        """Prompt length of every request of the file after the chat template is applied (``countPromptTokens``)."""
        from ..commands.infer import _text_of, parse_request_file
        body = json.loads(request) if isinstance(request, (str, bytes)) else request
        out = []
        for r in parse_request_file(body):
            text = self.template.apply(r["messages"], r["add_generation_prompt"], None, r["enable_thinking"]) if r["apply_chat_template"] \
                else _text_of(r["messages"])
            if self.llm.tokenizer is None:
                raise RuntimeError("count_prompt_tokens needs a tokenizer")
            out.append(len(self.llm.tokenizer.encode(text)))
        return out

    def capture_decoding_cuda_graph(self) -> bool:
        """Capture the decode graphs ahead of the first request: one per batch-size bucket the seat count can reach
        (``captureDecodingCUDAGraph``; ``cpp/runtime/llmRankRuntime.cpp:5326``).  False when graphs are switched off."""
        r, kv = self.llm.runner, self.llm.kv
        if not r.use_cuda_graphs or self.llm.engine is not None and self.llm.engine.status().resident > 0:
            return False
        seats = list(range(kv.max_seats))
        for s in seats:
            kv.free(s)
            kv.reserve(s, 8)
        try:
            for n in sorted({r.graph_bucket(k) for k in range(1, kv.max_seats + 1)}):
                r.decode_step_graph(seats[:n], [0] * n)
        finally:
            for s in seats:
                kv.free(s)
        return True

    def unavailable_reason(self) -> str:
        return self._unavailable

    def supports_stepped_execution(self) -> bool:
        return True

    def supports_seated_admission(self) -> bool:
        return self.llm.diffusion_decoder is None

    def max_batch_size(self) -> int:
        return int(self.llm.max_batch_size)

    def world_size(self) -> int:
        return int(self.llm.cfg.tp_size)

    def owns_global_rank(self, rank: int) -> bool:
        return int(rank) == int(self.llm.cfg.tp_rank)

    def has_draft_model(self) -> bool:
        return self.llm.spec_decoder is not None

    def open_session(self, enable_prefix_cache: bool = False):
        """The stepped-execution session a scheduler drives (``openSession``): admit / execute / release over this model."""
        from .session import ModelSession
        eos = self.llm.cfg.eos_token_id
        return ModelSession(self.llm.runner, eos if isinstance(eos, (list, tuple)) else [eos], enable_prefix_cache, self.llm.max_input_len,
                            self.llm.guided_vocab, spec_decoder=self.llm.spec_decoder)

    def get_generation_metrics(self) -> Dict[str, Any]:
        return dict(self._last)

    def get_scheduling_metrics(self):
        return self.llm.get_scheduling_metrics()

    def get_context_cache_metrics(self):
        return self.llm.get_context_cache_counters()

    def close(self) -> None:
        self.llm.close()
