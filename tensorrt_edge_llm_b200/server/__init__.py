"""OpenAI- and Anthropic-compatible HTTP serving over the in-flight-batching request engine.

Parity: ``tensorrt_edgellm/server/`` (``config.py`` dataclasses, ``runtime/engine.py`` ``LLM`` /
``SamplingParams``, ``runtime/engine_client.py`` admission control, ``api/routes.py``)."""
from ..runtime.llm import LLM, RequestOutput
from ..runtime.runner import SamplingParams
from .config import ApiConfig, ContextCacheConfig, ModelConfig, ServerConfig, SpeculativeConfig, parse_server_config

__all__ = ["LLM", "SamplingParams", "RequestOutput", "ApiConfig", "ContextCacheConfig", "ModelConfig", "ServerConfig",
           "SpeculativeConfig", "parse_server_config"]
