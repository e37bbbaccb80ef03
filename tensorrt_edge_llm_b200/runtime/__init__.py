"""Runtime: the generation façade (``LLM``, ``LLMRuntime``), the model runner and session, and — re-exported from the
native module — the request engine, handles, stream channels and scheduling options.

``tensorrt_edgellm.runtime`` resolves to this package, so the names of the reference's runtime module work unchanged:
``LLMRuntime``, ``RequestEngine``, ``RequestHandle``, ``StreamChannel``, ``MultiStageRuntime``, ``TTSRuntime``, ``TTS``,
``validate_scheduling_options`` (``python/nanobind/bindings.cpp:1359-1821``).  Attributes load lazily: importing the
package does not load the native module or torch-heavy submodules until a name is used."""
from __future__ import annotations

import importlib

_NATIVE = ("RequestEngine", "RequestHandle", "StreamChannel", "StreamChunk", "FinishReason", "EngineConfig", "EngineMetrics",
           "EngineStatus", "SchedulingOptions", "ResolvedSchedulingPolicy", "SessionCapabilities", "GenerationRequest",
           "RuntimeSession", "StepPlanner", "StepPlan", "validate_scheduling_options", "resolve_scheduling_policy", "Tokenizer",
           "ChatTemplate", "ChatMessage", "KVPageTable", "PrefixCache", "LLMEngineConfig", "ParallelConfig", "LoRAManager",
           "LLMInferenceRuntime", "LLMGenerationRequest", "LLMGenerationResponse", "GenerationEntry")
_LOCAL = {"LLM": ("llm", "LLM"), "LLMRuntime": ("facade", "LLMRuntime"), "SamplingParams": ("runner", "SamplingParams"),
          "ModelRunner": ("runner", "ModelRunner"), "ModelSession": ("session", "ModelSession"),
          "MultiStageRuntime": ("multistage", "MultiStageRuntime"), "KVCacheManager": ("kv_cache", "KVCacheManager"),
          "TTS": ("tts", "TTS"), "TTSRuntime": ("tts", "TTSRuntime"), "TTSSampling": ("tts", "TTSSampling")}

__all__ = sorted(_NATIVE + tuple(_LOCAL))


def __getattr__(name: str):
    if name in _LOCAL:
        mod, attr = _LOCAL[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    if name in _NATIVE:
        return getattr(importlib.import_module(f"{__name__}.native"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
