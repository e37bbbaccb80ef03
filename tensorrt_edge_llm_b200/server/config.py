"""Server configuration: dataclasses, validation and the ``serve`` argument parser.

Field names and defaults follow ``tensorrt_edgellm/server/config.py:112-404`` so a deployment's flags
carry over; there is no engine cache because nothing is compiled per model."""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence

DEFAULT_MAX_QUEUED_REQUESTS = 256


class ServerConfigError(ValueError):
    """A flag combination the runtime cannot honour."""


@dataclass
class SpeculativeConfig:
    method: str                                    # draft family; the draft checkpoint's own config decides the decoder and its head
    num_speculative_tokens: Optional[int] = None   # draft depth
    draft_model: str = ""
    draft_top_k: Optional[int] = None
    verify_tokens: Optional[int] = None

    def __post_init__(self):
        if self.method not in ("eagle3", "eagle4", "mtp", "dflash", "dflash2", "domino", "dspark", "lilicorr", "jetspec"):
            raise ServerConfigError(f"unknown speculative method {self.method!r}")
        for name in ("num_speculative_tokens", "draft_top_k", "verify_tokens"):
            v = getattr(self, name)
            if v is not None and v < 1:
                raise ServerConfigError(f"speculative_config.{name} must be at least 1")
        if self.verify_tokens is not None and self.verify_tokens > 128:
            raise ServerConfigError("speculative_config.verify_tokens is capped at 128")

    @classmethod
    def from_mapping(cls, raw: Mapping[str, Any]) -> "SpeculativeConfig":
        known = {"method", "num_speculative_tokens", "draft_model", "draft_top_k", "verify_tokens"}
        extra = set(raw) - known
        if extra:
            raise ServerConfigError(f"unknown speculative_config keys: {sorted(extra)}")
        return cls(**{k: raw[k] for k in raw})


@dataclass
class ContextCacheConfig:
    enabled: bool = False
    max_records: int = 1024
    max_snapshots: int = 0


@dataclass
class MultimodalConfig:
    max_image_tokens_per_image: int = 0
    max_image_tokens: int = 0
    encoder_cache_budget_bytes: int = 0


@dataclass
class ModelConfig:
    model: str
    max_input_len: int = 4096
    max_batch_size: int = 1
    max_kv_cache_capacity: int = 8192
    kv_cache_dtype: str = "auto"                   # auto (follow the checkpoint's kv_cache_quant) | fp8 | model
    speculative_config: Optional[SpeculativeConfig] = None
    context_cache_config: ContextCacheConfig = field(default_factory=ContextCacheConfig)
    multimodal_config: MultimodalConfig = field(default_factory=MultimodalConfig)
    enable_in_flight_batching: bool = False
    ifb_scheduling_mode: str = "auto"              # auto | mixed | prefill_first | single_cohort
    max_num_tokens: int = 0                        # 0 = runtime default
    max_chunk_tokens: int = 0
    scheduling_policy: str = "fcfs"                # fcfs | priority
    preemption: str = "none"                       # none | pause
    priority_reserved_slots: int = 0
    max_pause_steps: int = 0
    tensor_parallel_size: int = 1
    kv_page_size: int = 64
    device: str = ""
    tts_model: str = ""                            # directory of a speech pipeline (talker, code predictor, vocoder)

    def __post_init__(self):
        if self.max_batch_size < 1 or self.max_input_len < 1:
            raise ServerConfigError("max_batch_size and max_input_len must be positive")
        if self.max_kv_cache_capacity < self.max_input_len:
            raise ServerConfigError("max_kv_cache_capacity must hold at least max_input_len tokens")
        if self.ifb_scheduling_mode not in ("auto", "mixed", "prefill_first", "single_cohort"):
            raise ServerConfigError(f"unknown ifb_scheduling_mode {self.ifb_scheduling_mode!r}")
        if self.scheduling_policy not in ("fcfs", "priority"):
            raise ServerConfigError(f"unknown scheduling_policy {self.scheduling_policy!r}")
        if self.preemption not in ("none", "pause"):
            raise ServerConfigError(f"unknown preemption {self.preemption!r}")
        tuned = (self.ifb_scheduling_mode != "auto" or self.scheduling_policy != "fcfs" or self.preemption != "none"
                 or self.priority_reserved_slots or self.max_pause_steps or self.max_chunk_tokens)
        if tuned and not self.enable_in_flight_batching:
            raise ServerConfigError("scheduling options need --enable-in-flight-batching")
        if self.preemption == "pause" and self.scheduling_policy != "priority":
            raise ServerConfigError("--preemption pause needs --scheduling-policy priority")
        if self.priority_reserved_slots >= self.max_batch_size and self.priority_reserved_slots:
            raise ServerConfigError("priority_reserved_slots must leave at least one ordinary slot")

    def scheduling_dict(self) -> dict:
        d = {"mode": self.ifb_scheduling_mode, "policy": self.scheduling_policy, "preemption": self.preemption}
        if self.priority_reserved_slots:
            d["priority_reserved_slots"] = self.priority_reserved_slots
        if self.max_pause_steps:
            d["max_pause_steps"] = self.max_pause_steps
        if self.max_chunk_tokens:
            d["max_chunk_tokens"] = self.max_chunk_tokens
        if self.max_num_tokens:
            d["max_num_tokens"] = self.max_num_tokens
        return d


@dataclass
class ApiConfig:
    host: str = "0.0.0.0"
    port: int = 8000
    served_model_name: str = ""
    api_key: str = ""
    reasoning_parser: str = "auto"
    tool_call_parser: str = "auto"
    enable_auto_tool_choice: bool = False
    max_queued_requests: int = DEFAULT_MAX_QUEUED_REQUESTS
    queue_timeout: float = 600.0
    log_level: str = "info"
    min_request_priority: int = 0
    allowed_local_media_path: str = ""          # "" = requests may not name files of this machine

    def __post_init__(self):
        if not 0 < self.port < 65536:
            raise ServerConfigError("port must be in 1..65535")
        if self.max_queued_requests < 0 or self.queue_timeout <= 0:
            raise ServerConfigError("max_queued_requests must be >= 0 and queue_timeout positive")


@dataclass
class ServerConfig:
    model: ModelConfig
    api: ApiConfig


def create_argument_parser(prog: str = "trtedge serve") -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog=prog, description="Serve a checkpoint over OpenAI- and Anthropic-compatible HTTP routes")
    p.add_argument("model", help="checkpoint directory (Hugging Face layout, optionally quantised)")
    m = p.add_argument_group("model")
    m.add_argument("--max-input-len", type=int, default=4096)
    m.add_argument("--max-batch-size", type=int, default=1)
    m.add_argument("--max-kv-cache-capacity", type=int, default=8192)
    m.add_argument("--kv-cache-dtype", "--kv-cache-quantization", dest="kv_cache_dtype", default="auto", choices=["auto", "fp8", "model"],
                   help="KV page storage: fp8 = E4M3 bytes (half the memory per cached token); auto follows the checkpoint")
    m.add_argument("--enable-in-flight-batching", action="store_true")
    m.add_argument("--ifb-scheduling-mode", default="auto", choices=["auto", "mixed", "prefill_first", "single_cohort"])
    m.add_argument("--max-num-tokens", type=int, default=0)
    m.add_argument("--max-chunk-tokens", type=int, default=0)
    m.add_argument("--scheduling-policy", default="fcfs", choices=["fcfs", "priority"])
    m.add_argument("--preemption", default="none", choices=["none", "pause"])
    m.add_argument("--priority-reserved-slots", type=int, default=0)
    m.add_argument("--max-pause-steps", type=int, default=0)
    m.add_argument("--enable-context-cache", "--enable-context-reuse", dest="enable_context_cache", action="store_true",
                   help="share KV pages (and recurrent-state snapshots) between requests with a common prefix")
    m.add_argument("--context-cache-max-records", type=int, default=1024)
    m.add_argument("--context-cache-max-snapshots", type=int, default=0)
    m.add_argument("--max-image-tokens-per-image", type=int, default=0, help="cap on language-model rows one image may take (0 = tower default)")
    m.add_argument("--max-image-tokens", type=int, default=0, help="cap on image rows of one request (0 = max-input-len)")
    m.add_argument("--encoder-cache-budget-bytes", type=int, default=0, help="reuse encoder outputs of repeated media within this budget")
    for flag in ("--draft-top-k", "--spec-draft-step", "--spec-verify-tokens", "--spec-proposal-tokens", "--max-spec-verify-tokens",
                 "--max-spec-draft-tokens"):
        m.add_argument(flag, type=int, default=0, help="override of the matching --speculative-config field")
    for flag in ("--cache-dir", "--engine-cache-max-size-gb"):
        m.add_argument(flag, default="", help="accepted for command-line compatibility: checkpoints load directly, no engine is built or cached")
    m.add_argument("--clear-engine-cache", action="store_true", help="accepted for command-line compatibility (no engine cache exists)")
    m.add_argument("--speculative-config", default="", help='JSON, e.g. {"method": "eagle3", "draft_model": "<dir>"}')
    m.add_argument("--tensor-parallel-size", type=int, default=1)
    m.add_argument("--kv-page-size", type=int, default=64, choices=[64, 128])
    m.add_argument("--device", default="")
    m.add_argument("--tts-model", "--talker-engine-dir", dest="tts_model", default="",
                   help="directory of a speech pipeline; enables /v1/audio/speech and /v1/voices")
    a = p.add_argument_group("api")
    a.add_argument("--host", default="0.0.0.0")
    a.add_argument("--port", type=int, default=8000)
    a.add_argument("--served-model-name", default="")
    a.add_argument("--api-key", default="")
    a.add_argument("--reasoning-parser", default="auto")
    a.add_argument("--tool-call-parser", default="auto")
    a.add_argument("--enable-auto-tool-choice", action="store_true")
    a.add_argument("--max-queued-requests", type=int, default=DEFAULT_MAX_QUEUED_REQUESTS)
    a.add_argument("--queue-timeout", type=float, default=600.0)
    a.add_argument("--log-level", default="info")
    a.add_argument("--min-request-priority", type=int, default=0)
    a.add_argument("--allowed-local-media-path", default="", help="directory under which requests may name local media files; "
                   "without it only data: URIs are read")
    return p


def parse_server_config(argv: Optional[Sequence[str]] = None) -> ServerConfig:
    import json
    ns = create_argument_parser().parse_args(argv)
    spec = None
    if ns.speculative_config:
        try:
            spec = SpeculativeConfig.from_mapping(json.loads(ns.speculative_config))
        except json.JSONDecodeError as e:
            raise ServerConfigError(f"--speculative-config is not valid JSON: {e}") from None
    if spec is not None:
        # the reference's separate flags override single fields of the JSON
        for flag, names in (("draft_top_k", ("draft_top_k", "top_k")), ("spec_draft_step", ("num_speculative_tokens", "draft_steps")),
                            ("spec_verify_tokens", ("verify_tokens",)), ("max_spec_verify_tokens", ("verify_tokens",))):
            v = getattr(ns, flag)
            for name in names:
                if v and hasattr(spec, name):
                    setattr(spec, name, v)
    model = ModelConfig(
        model=ns.model, max_input_len=ns.max_input_len, max_batch_size=ns.max_batch_size,
        max_kv_cache_capacity=ns.max_kv_cache_capacity, kv_cache_dtype=getattr(ns, "kv_cache_dtype", "auto"), speculative_config=spec,
        context_cache_config=ContextCacheConfig(enabled=ns.enable_context_cache, max_records=ns.context_cache_max_records,
                                                max_snapshots=ns.context_cache_max_snapshots),
        multimodal_config=MultimodalConfig(ns.max_image_tokens_per_image, ns.max_image_tokens, ns.encoder_cache_budget_bytes),
        enable_in_flight_batching=ns.enable_in_flight_batching, ifb_scheduling_mode=ns.ifb_scheduling_mode,
        max_num_tokens=ns.max_num_tokens, max_chunk_tokens=ns.max_chunk_tokens, scheduling_policy=ns.scheduling_policy,
        preemption=ns.preemption, priority_reserved_slots=ns.priority_reserved_slots, max_pause_steps=ns.max_pause_steps,
        tensor_parallel_size=ns.tensor_parallel_size, kv_page_size=ns.kv_page_size, device=ns.device, tts_model=ns.tts_model)
    api = ApiConfig(host=ns.host, port=ns.port, served_model_name=ns.served_model_name, api_key=ns.api_key,
                    reasoning_parser=ns.reasoning_parser, tool_call_parser=ns.tool_call_parser,
                    enable_auto_tool_choice=ns.enable_auto_tool_choice, max_queued_requests=ns.max_queued_requests,
                    queue_timeout=ns.queue_timeout, log_level=ns.log_level, min_request_priority=ns.min_request_priority,
                    allowed_local_media_path=ns.allowed_local_media_path)
    return ServerConfig(model=model, api=api)
