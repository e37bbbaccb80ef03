"""Model, quantisation and parallel-mapping configuration.

Parses a Hugging Face ``config.json`` (plus ``hf_quant_config.json`` or an embedded
``quantization_config``) into the dataclasses the rest of the runtime consumes.

Parity: ``tensorrt_edgellm/config.py`` in the reference (``Mapping`` :365, ``QuantConfig`` :436,
``MambaConfig`` :528, ``GdnConfig`` :545, ``ModelConfig`` :629, ``ModelConfig.for_rank`` :1150,
``ModelConfig.from_pretrained`` :1199).  The field names a user touches are kept; the parsing
code is new and only covers what this runtime executes.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

# Quantisation type names (strings, so they survive a JSON round trip).
QUANT_NONE = "fp16"
QUANT_NVFP4 = "nvfp4"          # W4A4: NVFP4 weights, activations quantised dynamically
QUANT_NVFP4_A16 = "nvfp4_a16"  # W4A16: NVFP4 weights, 16-bit activations
QUANT_INT4_AWQ = "int4_awq"
QUANT_INT4_GPTQ = "int4_gptq"
QUANT_FP8 = "fp8"
QUANT_INT8_SQ = "int8_sq"
QUANT_MXFP8 = "mxfp8"
QUANT_Q8_0 = "q8_0"
# formats that are expanded to 16-bit when the checkpoint is loaded
EXPANDED_QUANT_TYPES = (QUANT_INT4_GPTQ, QUANT_FP8, QUANT_INT8_SQ, QUANT_MXFP8, QUANT_Q8_0)

NVFP4_BLOCK = 16
AWQ_GROUP = 128

LAYER_ATTENTION = "attention"
LAYER_MAMBA = "mamba"
LAYER_GDN = "gdn"
LAYER_MLP = "mlp"
LAYER_MOE = "moe"


@dataclass
class Mapping:
    """Tensor / expert parallel placement of one rank."""

    tp_size: int = 1
    tp_rank: int = 0
    ep_size: int = 1
    ep_rank: int = 0

    def __post_init__(self) -> None:
        if not (0 <= self.tp_rank < self.tp_size):
            raise ValueError(f"tp_rank {self.tp_rank} outside [0,{self.tp_size})")
        if not (0 <= self.ep_rank < self.ep_size):
            raise ValueError(f"ep_rank {self.ep_rank} outside [0,{self.ep_size})")

    @property
    def world_size(self) -> int:
        return max(self.tp_size, self.ep_size)


@dataclass
class QuantConfig:
    """How the linear layers of a checkpoint are stored."""

    quant_type: str = QUANT_NONE
    group_size: int = 1
    kv_cache_quant: Optional[str] = None            # None or "fp8"
    excluded: List[str] = field(default_factory=list)
    layer_overrides: Dict[str, str] = field(default_factory=dict)
    gptq_zero_point_offset: int = 1                 # GPTQ v1 checkpoints store zero - 1
    awq_layout: str = "modelopt"                    # "modelopt" (prepacked uint8) or "autoawq" (int32 qweight / qzeros / scales)
    quantize_activations: bool = True
    lm_head_quant_type: str = QUANT_NONE

    @property
    def is_quantized(self) -> bool:
        return self.quant_type != QUANT_NONE

    @property
    def uses_nvfp4_weights(self) -> bool:
        return self.quant_type in (QUANT_NVFP4, QUANT_NVFP4_A16)

    def module_quant_type(self, module_name: str) -> str:
        """Quantisation of one named linear (exclusions are glob-ish suffix patterns)."""
        if module_name in self.layer_overrides:
            return self.layer_overrides[module_name]
        for pat in self.excluded:
            p = pat.replace("*", "")
            if p and p in module_name:
                return QUANT_NONE
        return self.quant_type


@dataclass
class DiffusionConfig:
    """Block-diffusion generation parameters (``tensorrt_edgellm/config.py:576`` ``DiffusionConfig``): a canvas of
    ``canvas_length`` tokens is denoised with bidirectional attention for at most ``max_denoising_steps`` passes while the
    sampling temperature falls from ``t_max`` to ``t_min``; the entropy-bound sampler keeps the lowest-entropy positions
    whose summed entropy (all but the largest) stays within ``entropy_bound`` and re-noises the rest; a block has converged
    when every arg-max has been stable for more than ``stability_window`` passes and the mean entropy is below
    ``entropy_threshold``."""

    canvas_length: int = 256
    max_denoising_steps: int = 48
    t_max: float = 0.8
    t_min: float = 0.4
    sampler_type: str = "entropy_bound"
    entropy_bound: float = 0.1
    entropy_threshold: float = 0.005
    stability_window: int = 2
    self_conditioning_enabled: bool = True
    self_conditioning_size: int = 0

    @classmethod
    def from_hf(cls, hf: Dict[str, Any], gen: Optional[Dict[str, Any]] = None) -> "DiffusionConfig":
        gen = gen or {}
        own = hf.get("diffusion") or {}
        look = lambda k, d: own.get(k, gen.get(k, hf.get(k, d)))
        sampler = gen.get("sampler_config") or own.get("sampler_config") or {}
        name = str(sampler.get("_cls_name", own.get("sampler_type", "entropy_bound"))).lower().replace("_", "")
        return cls(canvas_length=int(look("canvas_length", 256)), max_denoising_steps=int(look("max_denoising_steps", 48)),
                   t_max=float(look("t_max", 0.8)), t_min=float(look("t_min", 0.4)),
                   sampler_type="entropy_bound" if "entropybound" in name else name,
                   entropy_bound=float(sampler.get("entropy_bound", look("entropy_bound", 0.1))),
                   entropy_threshold=float(sampler.get("entropy_threshold", look("entropy_threshold", 0.005))),
                   stability_window=int(sampler.get("stability_window", look("stability_window", 2))),
                   self_conditioning_enabled=bool(look("self_conditioning_enabled", True)),
                   self_conditioning_size=int(look("self_conditioning_size", 0) or 0))


@dataclass
class MambaConfig:
    """Mamba2 mixer geometry (Nemotron-H style)."""

    num_heads: int = 64
    head_dim: int = 64
    d_state: int = 128
    n_groups: int = 8
    conv_kernel: int = 4
    chunk_size: int = 128
    dt_limit: float = 50.0

    @property
    def intermediate_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def conv_dim(self) -> int:
        return self.intermediate_size + 2 * self.n_groups * self.d_state


@dataclass
class GdnConfig:
    """Gated-DeltaNet mixer geometry (Qwen3.5 style)."""

    num_k_heads: int = 16
    num_v_heads: int = 16
    head_k_dim: int = 128
    head_v_dim: int = 128
    conv_kernel: int = 4

    @property
    def key_dim(self) -> int:
        return self.num_k_heads * self.head_k_dim

    @property
    def value_dim(self) -> int:
        return self.num_v_heads * self.head_v_dim

    @property
    def conv_dim(self) -> int:
        return 2 * self.key_dim + self.value_dim


@dataclass
class ModelConfig:
    """Architecture description of a decoder (dense, MoE or hybrid)."""

    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    partial_rotary_factor: float = 1.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    has_qk_norm: bool = False
    attention_bias: bool = False
    attention_sink_bias: bool = False      # per-query-head learned sink logit joining every softmax denominator
    # Skip-softmax deployment (`skip_softmax.py`): per-length [[seqlen_bin, S], ...] tables, None = that phase runs dense
    skip_softmax_prefill_table: Optional[List[List[int]]] = None
    skip_softmax_decode_table: Optional[List[List[int]]] = None
    sliding_window: Optional[int] = None
    layer_windows: List[int] = field(default_factory=list)  # per layer: sliding window in tokens, 0 = full attention (empty = `sliding_window` everywhere)
    mrope_section: List[int] = field(default_factory=list)   # multimodal RoPE: rotary pairs per (temporal, height, width) component
    # KV-shared layers: the last `num_kv_shared_layers` layers project no keys / values of their own and attend over the cache of
    # a donor layer (the last layer before them with the same attention type).  `kv_donor_layers` overrides the rule per layer
    # (-1 = the layer's own cache).
    num_kv_shared_layers: int = 0
    # Gemma-4 style attention variants: full-attention layers take their values from the key projection (no v_proj), and
    # values pass a weightless per-head RMSNorm before they are cached
    attention_k_eq_v: bool = False
    has_value_norm: bool = False
    kv_donor_layers: List[int] = field(default_factory=list)
    rope_local_theta: float = 0.0                   # RoPE base of the sliding-window layers when it differs (Gemma 3)
    rope_local_scaling: Optional[Dict[str, Any]] = None
    query_pre_attn_scalar: float = 0.0              # attention scale = this ** -0.5 when set (Gemma), else head_dim ** -0.5
    final_logit_softcapping: float = 0.0
    hidden_act: str = "silu"
    dtype: str = "bfloat16"
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    shared_expert_intermediate_size: int = 0
    router_type: str = "softmax_topk"      # or "sigmoid_group_topk"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    # hybrid
    layer_types: List[str] = field(default_factory=list)   # mixer type per layer
    mlp_types: List[str] = field(default_factory=list)     # "mlp" / "moe" / "none" per layer
    mamba: Optional[MambaConfig] = None
    gdn: Optional[GdnConfig] = None
    diffusion: Optional[DiffusionConfig] = None      # block-diffusion checkpoints (model_type "diffusion_gemma")
    # draft heads
    draft_type: Optional[str] = None        # "eagle3" / "mtp"
    eagle3_target_hidden_size: int = 0
    eagle3_num_target_layers: int = 3
    eagle3_target_layer_ids: List[int] = field(default_factory=list)   # tapped target layers (default: low / mid / high)
    eagle3_norm_before_residual: bool = False
    # EAGLE-4 additions to the EAGLE-3 draft: one RMSNorm per tapped target layer in front of ``fc``, the final-norm output fed
    # back as the next step's feature, and a low-rank candidate head (``rank``-wide scores pick ``count`` tokens of the full
    # vocabulary, which are then scored exactly with their ``lm_head`` rows)
    eagle_fc_norm: bool = False
    eagle_norm_output: bool = False
    draft_candidate_rank: int = 0
    draft_candidate_count: int = 0
    draft_vocab_size: int = 0
    # DFlash block draft (draft_type "dflash"): tapped target layers, proposal block length, id of the mask token, and whether
    # row i's hidden state predicts position i + 1 (shifted labels) instead of its own position
    dflash_target_layer_ids: List[int] = field(default_factory=list)
    dflash_block_size: int = 16
    dflash_mask_token_id: int = 0
    dflash_shift_label: bool = False
    dflash_query_causal: bool = False       # JetSpec: block rows attend causally inside the block instead of to the whole block
    # Domino: a DFlash draft whose proposals after the first are corrected one by one by a small recurrent head over a shared
    # candidate pool (dflash_projector_type "domino")
    dflash_projector_type: str = ""
    # DFlash 2 (dflash_version 2): a dynamic grouped convolution around every sublayer of the block draft and a chain selector
    # (per-slot top-k candidates rescored against the token chosen for the slot before through two [V, rank] codebooks)
    dflash_version: int = 1
    dflash2_conv_kernel_size: int = 2
    dflash2_conv_group_size: int = 16
    dflash2_selector_rank: int = 256
    dflash2_selector_top_k: int = 16
    dflash2_output_multiplier: float = 1.0
    # DSpark (dflash_projector_type "dspark"): the block draft plus a rank-R bigram ("Markov") correction of its logits and an
    # optional confidence head that schedules the proposal length
    dspark_markov_rank: int = 0
    dspark_markov_head_type: str = ""
    dspark_enable_confidence_head: bool = False
    dspark_confidence_head_with_markov: bool = False
    # LiLiCorr (dflash_projector_type "lilicorr"): a small bidirectional transformer over the lattice of per-slot top-k
    # candidates that scores transitions between the candidates of consecutive slots
    lilicorr_candidate_topk: int = 0
    lilicorr_hidden_size: int = 0
    lilicorr_num_layers: int = 0
    lilicorr_num_heads: int = 0
    lilicorr_mlp_ratio: float = 0.0
    lilicorr_factor_dim: int = 0
    lilicorr_vector_eps: float = 0.0
    lilicorr_logit_scale: float = 0.0
    domino_pool_size: int = 2048
    domino_proj_dim: int = 256
    domino_gru_hidden_dim: int = 256
    # quant / parallel
    quant: QuantConfig = field(default_factory=QuantConfig)
    mapping: Mapping = field(default_factory=Mapping)
    bos_token_id: Optional[int] = None
    eos_token_id: Any = None

    def __post_init__(self) -> None:
        if self.num_attention_heads % max(self.num_key_value_heads, 1):
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if not self.layer_types:
            self.layer_types = [LAYER_ATTENTION] * self.num_hidden_layers
        if not self.mlp_types:
            kind = LAYER_MOE if self.num_experts > 0 else LAYER_MLP
            self.mlp_types = [kind] * self.num_hidden_layers
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types length must equal num_hidden_layers")

    # -- derived ---------------------------------------------------------------------------
    @property
    def tp_size(self) -> int:
        return self.mapping.tp_size

    @property
    def tp_rank(self) -> int:
        return self.mapping.tp_rank

    @property
    def compute_dtype(self) -> torch.dtype:
        return {"bfloat16": torch.bfloat16, "float16": torch.float16,
                "float32": torch.float32}[self.dtype]

    def kv_donor(self, layer_idx: int) -> int:
        """The layer whose KV cache ``layer_idx`` attends over, or -1 when it writes and reads its own."""
        if self.kv_donor_layers:
            d = int(self.kv_donor_layers[layer_idx])
            if d >= layer_idx:
                raise ValueError(f"layer {layer_idx}: a KV donor must be an earlier layer, got {d}")
            return d
        n = int(self.num_kv_shared_layers or 0)
        first = self.num_hidden_layers - n
        if n <= 0 or layer_idx < first:
            return -1
        if first <= 0:
            raise ValueError("num_kv_shared_layers leaves no layer with keys and values of its own")
        kind = lambda i: bool(self.layer_windows[i]) if self.layer_windows else False
        for d in range(first - 1, -1, -1):
            if kind(d) == kind(layer_idx) and (not self.layer_types or self.layer_types[d] == LAYER_ATTENTION):
                return d
        raise ValueError(f"layer {layer_idx} shares KV but no earlier layer has its attention type")

    @property
    def is_eagle4_draft(self) -> bool:
        return self.draft_type == "eagle3" and (self.eagle_fc_norm or self.eagle_norm_output or self.draft_candidate_count > 0)

    @property
    def is_hybrid(self) -> bool:
        return any(t != LAYER_ATTENTION for t in self.layer_types)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def num_attn_layers(self) -> int:
        return sum(t == LAYER_ATTENTION for t in self.layer_types)

    @property
    def num_mamba_layers(self) -> int:
        return sum(t == LAYER_MAMBA for t in self.layer_types)

    @property
    def num_gdn_layers(self) -> int:
        return sum(t == LAYER_GDN for t in self.layer_types)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    def for_rank(self, rank: int, world: int, ep: bool = False) -> "ModelConfig":
        """Copy of this config placed on ``rank`` of ``world`` (TP, or EP when ``ep``)."""
        cfg = dataclasses.replace(self)
        cfg.quant = dataclasses.replace(self.quant)
        if ep:      # attention and dense projections tensor-parallel, experts sharded by expert id
            if self.num_attention_heads % world or self.num_experts % world:
                raise ValueError(f"{self.num_attention_heads} heads / {self.num_experts} experts not divisible by {world} ranks")
            cfg.mapping = Mapping(tp_size=world, tp_rank=rank, ep_size=world, ep_rank=rank)
        else:
            if self.num_attention_heads % world:
                raise ValueError(f"{self.num_attention_heads} heads not divisible by TP {world}")
            cfg.mapping = Mapping(tp_size=world, tp_rank=rank)
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        d = dict(d)
        if isinstance(d.get("quant"), dict):
            d["quant"] = QuantConfig(**d["quant"])
        if isinstance(d.get("mapping"), dict):
            d["mapping"] = Mapping(**d["mapping"])
        if isinstance(d.get("mamba"), dict):
            d["mamba"] = MambaConfig(**d["mamba"])
        if isinstance(d.get("gdn"), dict):
            d["gdn"] = GdnConfig(**d["gdn"])
        if isinstance(d.get("diffusion"), dict):
            d["diffusion"] = DiffusionConfig(**d["diffusion"])
        known = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})

    # -- HF parsing ------------------------------------------------------------------------
    @classmethod
    def from_hf_dict(cls, hf: Dict[str, Any], quant: Optional[QuantConfig] = None,
                     has_qk_norm: Optional[bool] = None) -> "ModelConfig":
        llm = hf.get("text_config", hf)
        model_type = llm.get("model_type", hf.get("model_type", "llama"))
        heads = int(llm["num_attention_heads"])
        hidden = int(llm["hidden_size"])
        head_dim = int(llm.get("head_dim") or hidden // heads)
        rope_theta = llm.get("rope_theta")
        rope_scaling = llm.get("rope_scaling") or llm.get("rope_parameters")
        if rope_theta is None and isinstance(rope_scaling, dict):
            rope_theta = rope_scaling.get("rope_theta")
        mrope_section = list((rope_scaling or {}).get("mrope_section") or []) if isinstance(rope_scaling, dict) else []
        if isinstance(rope_scaling, dict) and rope_scaling.get("rope_type", rope_scaling.get("type")) in (None, "default", "mrope"):
            rope_scaling = None
        n_layers = int(llm["num_hidden_layers"])
        layer_types, mlp_types, mamba, gdn = _parse_hybrid(llm, n_layers)
        if has_qk_norm is None:
            has_qk_norm = model_type in ("qwen3", "qwen3_moe", "qwen3_next", "qwen3_5")
        torch_dtype = str(llm.get("torch_dtype", llm.get("dtype", "bfloat16"))).replace("torch.", "")
        if torch_dtype not in ("bfloat16", "float16", "float32"):
            torch_dtype = "bfloat16"
        extra: Dict[str, Any] = {}
        if str(model_type).startswith("gemma") or model_type == "diffusion_gemma":
            extra = _parse_gemma(llm, n_layers)
            if model_type == "diffusion_gemma":
                extra["diffusion"] = DiffusionConfig.from_hf(hf, hf.get("generation_config"))
            rope_theta, rope_scaling = extra.pop("rope_theta", rope_theta), extra.pop("rope_scaling", rope_scaling)
            layer_types = []
        router = "sigmoid_group_topk" if model_type in ("nemotron_h", "deepseek_v3") and llm.get("n_routed_experts") else "softmax_topk"
        from .skip_softmax import resolve as _resolve_skip_softmax
        skip = _resolve_skip_softmax(hf, llm if llm is not hf else None)
        family_extra = bool(extra)            # family-specific fields parsed above (they decide the sliding-window rule below)
        extra.setdefault("skip_softmax_prefill_table", skip.prefill_table)
        extra.setdefault("skip_softmax_decode_table", skip.decode_table)
        cfg = cls(
            model_type=model_type,
            vocab_size=int(llm["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(llm.get("intermediate_size", 4 * hidden)),
            num_hidden_layers=n_layers,
            num_attention_heads=heads,
            num_key_value_heads=int(llm.get("num_key_value_heads", heads)),
            head_dim=head_dim,
            rms_norm_eps=float(llm.get("rms_norm_eps", llm.get("layer_norm_epsilon", 1e-6))),
            rope_theta=float(rope_theta if rope_theta is not None else 10000.0),
            rope_scaling=rope_scaling,
            mrope_section=mrope_section,
            partial_rotary_factor=float(llm.get("partial_rotary_factor", 1.0)),
            max_position_embeddings=int(llm.get("max_position_embeddings", 32768)),
            tie_word_embeddings=bool(hf.get("tie_word_embeddings", llm.get("tie_word_embeddings", False))),
            has_qk_norm=bool(has_qk_norm),
            attention_bias=bool(llm.get("attention_bias", str(model_type).startswith("qwen2"))),     # Qwen2 family (text, MoE, VL): q/k/v carry a bias
            attention_sink_bias=bool(llm.get("attention_sink_bias", False)),
            sliding_window=llm.get("sliding_window") if (llm.get("use_sliding_window", False) or family_extra) else None,
            hidden_act=llm.get("hidden_activation") or llm.get("hidden_act", llm.get("mlp_hidden_act", "silu")),
            **extra,
            dtype=torch_dtype,
            num_experts=int(llm.get("num_experts") or llm.get("num_local_experts") or llm.get("n_routed_experts") or 0),
            num_experts_per_tok=int(llm.get("num_experts_per_tok", 0) or 0),
            moe_intermediate_size=int(llm.get("moe_intermediate_size", 0) or 0),
            norm_topk_prob=bool(llm.get("norm_topk_prob", True)),
            shared_expert_intermediate_size=int(llm.get("shared_expert_intermediate_size", llm.get("moe_shared_expert_intermediate_size", 0)) or 0),
            router_type=router,
            n_group=int(llm.get("n_group", 1) or 1),
            topk_group=int(llm.get("topk_group", 1) or 1),
            routed_scaling_factor=float(llm.get("routed_scaling_factor", 1.0) or 1.0),
            layer_types=layer_types,
            mlp_types=mlp_types,
            mamba=mamba,
            gdn=gdn,
            quant=quant or QuantConfig(),
            bos_token_id=llm.get("bos_token_id"),
            eos_token_id=llm.get("eos_token_id"),
            draft_type="dflash" if (llm.get("dflash_config") or llm.get("jetspec_config")
                                    or any(k in str(hf.get("architectures", "")).lower() for k in ("dflash", "jetspec", "domino"))) else (
                "eagle3" if (llm.get("draft_vocab_size") or "eagle" in str(hf.get("architectures", "")).lower()
                             or hf.get("speculators_model_type") == "eagle3"
                             or (any(llm.get(k) for k in _EAGLE4_KEYS) and (hf.get("eagle_config") or {}).get("use_aux_hidden_state"))) else None),
            dflash_target_layer_ids=list((llm.get("dflash_config") or {}).get("target_layer_ids", []) or []),
            dflash_block_size=int((llm.get("dflash_config") or {}).get("block_size", llm.get("block_size", 16)) or 16),
            dflash_mask_token_id=int((llm.get("dflash_config") or {}).get("mask_token_id", llm.get("mask_token_id", 0)) or 0),
            dflash_shift_label=bool((llm.get("dflash_config") or {}).get("shift_label", llm.get("dflash_shift_label", False))),
            dflash_query_causal=bool((llm.get("dflash_config") or llm.get("jetspec_config") or {}).get("query_causal", llm.get("dflash_query_causal", False))),
            domino_pool_size=int((llm.get("dflash_config") or {}).get("pool_size", llm.get("domino_pool_size", 2048)) or 2048),
            domino_proj_dim=int((llm.get("dflash_config") or {}).get("proj_dim", llm.get("domino_proj_dim", 256)) or 256),
            domino_gru_hidden_dim=int((llm.get("dflash_config") or {}).get("gru_hidden_dim", llm.get("domino_gru_hidden_dim", 256)) or 256),
            **{"dflash_projector_type": str((llm.get("dflash_config") or {}).get("projector_type", llm.get("dflash_projector_type", "")) or ""),
               **_parse_dflash2(llm, hf)},
            num_kv_shared_layers=int(llm.get("num_kv_shared_layers", 0) or 0),
            attention_k_eq_v=bool(llm.get("attention_k_eq_v", False)),
            has_value_norm=bool(llm.get("has_value_norm", llm.get("use_value_norm", False))),
            draft_vocab_size=int(llm.get("draft_vocab_size", 0) or 0),
            eagle3_target_hidden_size=int(llm.get("target_hidden_size", 0) or 0),
            eagle3_norm_before_residual=bool(llm.get("norm_before_residual", False)),
            **{"eagle3_target_layer_ids": list((hf.get("eagle_config") or {}).get("eagle_aux_hidden_state_layer_ids", []) or []),
               **_parse_eagle4(llm, hf)},
        )
        for key, value in _parse_dspark(llm, hf).items():
            setattr(cfg, key, value)
        return cfg

    @classmethod
    def from_pretrained(cls, model_dir: str, mapping: Optional[Mapping] = None) -> "ModelConfig":
        hf = load_config_dict(model_dir)
        gen_path = os.path.join(model_dir, "generation_config.json")
        if hf.get("model_type") == "diffusion_gemma" and os.path.exists(gen_path) and "generation_config" not in hf:
            with open(gen_path, "r", encoding="utf-8") as f:
                hf["generation_config"] = json.load(f)
        quant = parse_quant_config(model_dir, hf)
        cfg = cls.from_hf_dict(hf, quant=quant, has_qk_norm=_detect_qk_norm(model_dir, hf))
        if mapping is not None:
            cfg.mapping = mapping
        return cfg


# ------------------------------------------------------------------------------------------

def load_config_dict(model_dir: str) -> Dict[str, Any]:
    """Read ``config.json`` of a checkpoint directory."""
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        return json.load(f)


def load_checkpoint_config_dicts(model_dir: str) -> Dict[str, Dict[str, Any]]:
    """All JSON side files a checkpoint may carry, keyed by role."""
    out: Dict[str, Dict[str, Any]] = {"config": load_config_dict(model_dir)}
    for role, name in (("quant", "hf_quant_config.json"), ("generation", "generation_config.json"),
                       ("tokenizer", "tokenizer_config.json")):
        p = os.path.join(model_dir, name)
        if os.path.exists(p):
            with open(p, "r", encoding="utf-8") as f:
                out[role] = json.load(f)
    return out


_ALGO_TO_QUANT = {
    "NVFP4": QUANT_NVFP4, "NVFP4_AWQ": QUANT_NVFP4, "W4A16_NVFP4": QUANT_NVFP4_A16,
    "W4A16_AWQ": QUANT_INT4_AWQ, "INT4_AWQ": QUANT_INT4_AWQ, "W4A16": QUANT_INT4_AWQ,
    "W4A16_GPTQ": QUANT_INT4_GPTQ, "FP8": QUANT_FP8, "FP8_PER_CHANNEL_PER_TOKEN": QUANT_FP8,
    "W8A8_SQ_PER_CHANNEL": QUANT_INT8_SQ, "INT8_SQ": QUANT_INT8_SQ, "INT8_SMOOTHQUANT": QUANT_INT8_SQ,
    "MXFP8": QUANT_MXFP8, "Q8_0": QUANT_Q8_0,
}


def parse_quant_config(model_dir: str, hf: Optional[Dict[str, Any]] = None) -> QuantConfig:
    """Detect the quantisation of a checkpoint.

    Understands ModelOpt (``hf_quant_config.json`` with ``quant_algo`` / ``kv_cache_quant_algo`` /
    ``exclude_modules``), AutoAWQ / GPTQ ``quantization_config`` blocks and compressed-tensors
    ``config_groups``.  Parity: ``tensorrt_edgellm/config.py:3216-3425``.
    """
    hf = hf if hf is not None else load_config_dict(model_dir)
    p = os.path.join(model_dir, "hf_quant_config.json")
    qc: Dict[str, Any] = {}
    if os.path.exists(p):
        with open(p, "r", encoding="utf-8") as f:
            qc = json.load(f).get("quantization", {})
    elif isinstance(hf.get("quantization_config"), dict):
        qc = hf["quantization_config"]
    if not qc:
        return QuantConfig()
    algo = str(qc.get("quant_algo") or "").upper()
    method = str(qc.get("quant_method") or "").lower()
    quant_type = QUANT_NONE
    group = 1
    if algo in _ALGO_TO_QUANT:
        quant_type = _ALGO_TO_QUANT[algo]
    elif method == "awq":
        quant_type = QUANT_INT4_AWQ
    elif method == "gptq":
        quant_type = QUANT_INT4_GPTQ
    elif method == "fp8":
        quant_type = QUANT_FP8
    elif method == "modelopt" and "NVFP4" in str(qc).upper():
        quant_type = QUANT_NVFP4
    elif "config_groups" in qc:
        for grp in qc["config_groups"].values():
            w = grp.get("weights", {})
            if w.get("num_bits") == 4 and w.get("type") == "float":
                quant_type = QUANT_NVFP4 if grp.get("input_activations") else QUANT_NVFP4_A16
            elif w.get("num_bits") == 4:
                quant_type = QUANT_INT4_AWQ
                group = int(w.get("group_size", AWQ_GROUP))
            elif w.get("num_bits") == 8 and w.get("type") == "float":
                quant_type = QUANT_FP8
    if quant_type in (QUANT_NVFP4, QUANT_NVFP4_A16):
        group = NVFP4_BLOCK
    elif quant_type in (QUANT_INT4_AWQ, QUANT_INT4_GPTQ):
        group = int(qc.get("group_size", qc.get("q_group_size", AWQ_GROUP)))
    kv = qc.get("kv_cache_quant_algo") or (qc.get("kv_cache_scheme") and "fp8")
    kv = "fp8" if kv and "FP8" in str(kv).upper() else None
    excluded = list(qc.get("exclude_modules") or qc.get("ignore") or qc.get("modules_to_not_convert") or [])
    return QuantConfig(quant_type=quant_type, group_size=group, kv_cache_quant=kv, excluded=excluded,
                       awq_layout="autoawq" if method == "awq" else "modelopt",
                       gptq_zero_point_offset=0 if str(qc.get("checkpoint_format", "gptq")).lower() == "gptq_v2" else 1)


def _checkpoint_keys(model_dir: str) -> List[str]:
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx, "r", encoding="utf-8") as f:
            return list(json.load(f).get("weight_map", {}).keys())
    p = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(p):
        from .checkpoint.safetensors_io import SafetensorsFile
        return SafetensorsFile(p).keys()
    return []


def _detect_qk_norm(model_dir: str, hf: Dict[str, Any]) -> Optional[bool]:
    keys = _checkpoint_keys(model_dir)
    if not keys:
        return None
    return any(k.endswith("self_attn.q_norm.weight") for k in keys)


def _parse_gemma(llm: Dict[str, Any], n_layers: int) -> Dict[str, Any]:
    """Gemma 2 / 3 text decoders: alternating sliding-window and full-attention layers with their own RoPE bases."""
    # Gemma 3n / 4 checkpoints add pieces this decoder does not have; refuse them by name instead of loading them as Gemma 3
    missing = []
    gh = llm.get("global_head_dim")
    if gh and int(gh) != int(llm.get("head_dim") or gh):
        missing.append("full-attention layers with a head size of their own (global_head_dim)")
    if llm.get("num_global_key_value_heads") and int(llm["num_global_key_value_heads"]) != int(llm.get("num_key_value_heads") or 0):
        missing.append("full-attention layers with a KV head count of their own (num_global_key_value_heads)")
    if int(llm.get("hidden_size_per_layer_input") or 0) > 0:
        missing.append("per-layer input embeddings inside the decoder (hidden_size_per_layer_input)")
    if llm.get("altup_num_inputs") or llm.get("laurel_rank"):
        missing.append("AltUp / LAuReL blocks")
    if int(llm.get("num_experts") or 0) > 0 or llm.get("enable_moe_block"):
        missing.append("the Gemma mixture-of-experts block")
    if missing:
        raise NotImplementedError(f"{llm.get('model_type', 'gemma')}: this checkpoint needs " + "; ".join(missing) +
                                  ", which the Gemma decoder here does not build")
    win = int(llm.get("sliding_window") or 0)
    kinds = llm.get("layer_types")
    if not kinds:
        pat = int(llm.get("sliding_window_pattern", 6) or 6)
        kinds = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(n_layers)]
    out: Dict[str, Any] = {"layer_windows": [win if "sliding" in str(k) else 0 for k in kinds],
                           "query_pre_attn_scalar": float(llm.get("query_pre_attn_scalar") or 0.0),
                           "final_logit_softcapping": float(llm.get("final_logit_softcapping") or 0.0)}
    rp = llm.get("rope_parameters") or {}
    full, local = rp.get("full_attention"), rp.get("sliding_attention")
    if isinstance(full, dict):
        out["rope_theta"] = full.get("rope_theta", 1e6)
        out["rope_scaling"] = None if full.get("rope_type", "default") == "default" else full
        out["rope_local_theta"] = float((local or {}).get("rope_theta", 1e4))
        out["rope_local_scaling"] = None if (local or {}).get("rope_type", "default") == "default" else local
    else:
        out["rope_local_theta"] = float(llm.get("rope_local_base_freq", 0.0) or 0.0)
    if llm.get("attn_logit_softcapping"):
        raise ValueError("attention logit soft-capping (Gemma 2) is not supported by the attention kernels")
    return out


def _parse_dspark(llm: dict, hf: dict) -> dict:
    """DSpark draft fields (``dspark_config``, a top-level ``markov_head_type`` or an architecture named ``…DSparkModel``;
    ``tensorrt_edgellm/config.py:1880-1905``): the block geometry may sit at the top level instead of in ``dflash_config``, labels
    are shifted by default, the Markov head is of type ``vanilla`` with a positive rank."""
    archs = [str(a) for a in list(hf.get("architectures") or []) + list(llm.get("architectures") or [])]
    d = hf.get("dspark_config") or llm.get("dspark_config") or {}
    if not (d or llm.get("markov_head_type") or any(a.endswith("DSparkModel") for a in archs)):
        return {}
    f = hf.get("dflash_config") or llm.get("dflash_config") or {}
    look = lambda key, default: d.get(key, f.get(key, llm.get(key, hf.get(key, default))))
    head = str(look("markov_head_type", "") or "vanilla")
    if head != "vanilla":
        raise ValueError(f"DSpark supports markov_head_type 'vanilla' only, got {head!r}")
    rank = int(look("markov_rank", 0) or 0)
    if rank <= 0:
        raise ValueError("DSpark requires a positive markov_rank")
    block = int(look("block_size", 7))
    if block < 2:
        raise ValueError(f"DSpark block_size must be at least 2, got {block}")
    return {"draft_type": "dflash", "dflash_projector_type": "dspark", "dflash_block_size": block,
            "dflash_mask_token_id": int(look("mask_token_id", 0) or 0),
            "dflash_target_layer_ids": [int(i) for i in (look("target_layer_ids", []) or [])],
            "dflash_shift_label": bool(look("shift_label", True)),
            "dflash_query_causal": bool(d.get("causal", llm.get("dflash_query_causal", f.get("causal", False)))),
            "dspark_markov_rank": rank, "dspark_markov_head_type": head,
            "dspark_enable_confidence_head": bool(look("enable_confidence_head", False)),
            "dspark_confidence_head_with_markov": bool(look("confidence_head_with_markov", False))}


_LILICORR_FIELDS = ("lilicorr_candidate_topk", "lilicorr_hidden_size", "lilicorr_num_layers", "lilicorr_num_heads", "lilicorr_mlp_ratio",
                    "lilicorr_factor_dim", "lilicorr_vector_eps", "lilicorr_logit_scale")


def _parse_dflash2(llm: dict, hf: dict) -> dict:
    """DFlash 2 fields of a draft checkpoint (architecture ``DFlash2DraftModel``) with the reference's rules
    (``tensorrt_edgellm/dflash.py:262-305``): block size 2..16, non-causal blocks, unique tapped layers, the convolution and
    selector sizes spelled out in ``dflash_config``."""
    archs = {str(a) for a in list(hf.get("architectures") or []) + list(llm.get("architectures") or [])}
    f = {**(hf.get("dflash_config") or {}), **(llm.get("dflash_config") or {})}
    projector = str(f.get("projector_type", "") or "") or ("lilicorr" if "LiLiCorrDraftModel" in archs else "")
    lilicorr = projector == "lilicorr"
    if "DFlash2DraftModel" not in archs and not lilicorr:
        return {}
    extra = {}
    if lilicorr:
        if not f.get("lilicorr_enabled", False):
            raise ValueError("LiLiCorr requires dflash_config.lilicorr_enabled=true")
        missing = [n for n in _LILICORR_FIELDS if n not in f]
        if missing:
            raise ValueError(f"LiLiCorr requires dflash_config.{', '.join(missing)}")
        extra = {n: (float(f[n]) if n in ("lilicorr_mlp_ratio", "lilicorr_vector_eps", "lilicorr_logit_scale") else int(f[n]))
                 for n in _LILICORR_FIELDS}
        k = extra["lilicorr_candidate_topk"]
        if k <= 0 or k > 16 or k & (k - 1):
            raise ValueError(f"LiLiCorr lilicorr_candidate_topk must be a power of two <= 16, got {k}")
        for n, v in extra.items():
            if not v > 0:
                raise ValueError(f"LiLiCorr {n} must be positive, got {v}")
        if not (f.get("target_layer_ids") or llm.get("target_layer_ids")):
            raise ValueError("LiLiCorr requires at least one target-layer ID")
        extra["dflash_projector_type"] = "lilicorr"
    for name in ("conv_kernel_size", "conv_group_size") + (() if lilicorr else ("selector_rank", "selector_top_k")):
        if name not in f:
            raise ValueError(f"DFlash V2 requires dflash_config.{name}")
    causal = f.get("is_causal", llm.get("is_causal", hf.get("is_causal")))
    if causal is None:
        raise ValueError("DFlash V2 requires is_causal")
    if causal:
        raise ValueError("DFlash V2 draft checkpoint requires is_causal=false")
    block = int(f.get("block_size", llm.get("block_size", 16)))
    if not 2 <= block <= 16:
        raise ValueError(f"DFlash V2 block_size must be in [2, 16], got {block}")
    ids = list(f.get("target_layer_ids") or llm.get("target_layer_ids") or [])
    if len(set(ids)) != len(ids):
        raise ValueError("DFlash V2 target-layer IDs must be unique")
    taps, group = int(f["conv_kernel_size"]), int(f["conv_group_size"])
    if not 1 <= taps <= 4 or group < 2 or group % 2:
        raise ValueError("DFlash V2 convolution: 1 to 4 taps and an even group size")
    if not lilicorr and (not 1 <= int(f["selector_top_k"]) <= 32 or not 1 <= int(f["selector_rank"]) <= 1024):
        raise ValueError("DFlash V2 selector: at most 32 candidates per slot and rank 1024")
    mult = f.get("output_multiplier")
    if mult is not None and not float(mult) > 0:
        raise ValueError(f"DFlash V2 output_multiplier must be positive, got {mult}")
    return {"dflash_version": 2, "dflash2_conv_kernel_size": taps, "dflash2_conv_group_size": group,
            "dflash2_selector_rank": int(f.get("selector_rank", 0) or 0), "dflash2_selector_top_k": int(f.get("selector_top_k", 0) or 0),
            "dflash2_output_multiplier": float(mult) if mult is not None else 1.0, **extra}


_EAGLE4_KEYS = ("fc_norm", "norm_output", "efficient_lm_head_config")
_MAX_CANDIDATES, _MAX_CANDIDATE_RANK = 1024, 1024


def _parse_eagle4(llm: dict, hf: dict) -> dict:
    """EAGLE-4 draft switches of a checkpoint config (``fc_norm``, ``norm_output``, ``efficient_lm_head_config``) with the
    reference's consistency rules (``tensorrt_edgellm/config.py:2401-2462``): a candidate head is of type ``low_rank``, needs
    ``norm_output``, scores the full vocabulary and excludes logit soft-capping; none of the switches combines with
    ``norm_before_residual``."""
    if not any(llm.get(k) for k in _EAGLE4_KEYS):
        return {}
    if llm.get("norm_before_residual") or llm.get("norm_before_fc"):
        raise ValueError("EAGLE drafts with fc_norm, norm_output or a candidate head do not support norm_before_residual / norm_before_fc")
    out = {"eagle_fc_norm": bool(llm.get("fc_norm", False)), "eagle_norm_output": bool(llm.get("norm_output", False))}
    ids = (llm.get("eagle_aux_hidden_state_layer_ids") or (hf.get("eagle_config") or {}).get("eagle_aux_hidden_state_layer_ids")
           or llm.get("target_layer_ids") or [])
    n_aux = llm.get("num_aux_hidden_states")
    if n_aux is not None and ids and int(n_aux) != len(ids):
        raise ValueError(f"EAGLE draft num_aux_hidden_states={n_aux} does not match its {len(ids)} tapped layers")
    if ids:
        out["eagle3_target_layer_ids"] = [int(i) for i in ids]
        out["eagle3_num_target_layers"] = len(ids)
    elif n_aux:
        out["eagle3_num_target_layers"] = int(n_aux)
    head = llm.get("efficient_lm_head_config")
    if head:
        if head.get("type") != "low_rank":
            raise ValueError(f"EAGLE candidate head type {head.get('type')!r} is not supported; expected 'low_rank'")
        vocab = int(llm["vocab_size"])
        count, rank = int(head.get("num_candidates", 0) or 0), int(head.get("rank", 0) or 0)
        if not 0 < count <= min(vocab, _MAX_CANDIDATES):
            raise ValueError(f"EAGLE candidate head num_candidates={count} must be in [1, {min(vocab, _MAX_CANDIDATES)}]")
        if not 0 < rank <= _MAX_CANDIDATE_RANK or rank % 8:
            raise ValueError(f"EAGLE candidate head rank={rank} must be a multiple of 8 in [8, {_MAX_CANDIDATE_RANK}]")
        if not out["eagle_norm_output"]:
            raise ValueError("an EAGLE candidate head requires norm_output=true")
        if llm.get("final_logit_softcapping") is not None:
            raise ValueError("an EAGLE candidate head does not support final_logit_softcapping")
        dv = llm.get("draft_vocab_size")
        if dv is not None and int(dv) != vocab:
            raise ValueError(f"an EAGLE candidate head scores the full vocabulary; draft_vocab_size={dv} must equal vocab_size={vocab}")
        out["draft_candidate_rank"], out["draft_candidate_count"] = rank, count
    return out


def _parse_hybrid(llm: Dict[str, Any], n_layers: int):
    """Per-layer mixer / MLP kinds for hybrid checkpoints (Nemotron-H pattern string or HF
    ``layer_types`` / ``layers_block_type`` lists)."""
    layer_types: List[str] = []
    mlp_types: List[str] = []
    mamba = gdn = None
    pattern = llm.get("hybrid_override_pattern")
    raw = llm.get("layers_block_type") or llm.get("layer_types")
    if pattern:
        # Nemotron-H: one character per block: M = mamba, * = attention, - = MLP, E = MoE.
        for ch in pattern:
            if ch == "M":
                layer_types.append(LAYER_MAMBA); mlp_types.append("none")
            elif ch == "*":
                layer_types.append(LAYER_ATTENTION); mlp_types.append("none")
            elif ch == "-":
                layer_types.append("none"); mlp_types.append(LAYER_MLP)
            elif ch == "E":
                layer_types.append("none"); mlp_types.append(LAYER_MOE)
    elif raw:
        for t in raw:
            t = str(t).lower()
            if "mamba" in t:
                layer_types.append(LAYER_MAMBA)
            elif "linear" in t or "gdn" in t or "delta" in t:
                layer_types.append(LAYER_GDN)
            else:
                layer_types.append(LAYER_ATTENTION)
    if any(t == LAYER_MAMBA for t in layer_types):
        mamba = MambaConfig(
            num_heads=int(llm.get("mamba_num_heads", 64)), head_dim=int(llm.get("mamba_head_dim", 64)),
            d_state=int(llm.get("ssm_state_size", llm.get("mamba_d_state", 128))),
            n_groups=int(llm.get("n_groups", llm.get("mamba_n_groups", 8))),
            conv_kernel=int(llm.get("conv_kernel", llm.get("mamba_d_conv", 4))),
            chunk_size=int(llm.get("chunk_size", llm.get("mamba_chunk_size", 128))))
    if any(t == LAYER_GDN for t in layer_types):
        gdn = GdnConfig(
            num_k_heads=int(llm.get("linear_num_key_heads", 16)), num_v_heads=int(llm.get("linear_num_value_heads", 16)),
            head_k_dim=int(llm.get("linear_key_head_dim", 128)), head_v_dim=int(llm.get("linear_value_head_dim", 128)),
            conv_kernel=int(llm.get("linear_conv_kernel_dim", 4)))
    if layer_types and len(layer_types) != n_layers:
        layer_types, mlp_types = [], []
    if layer_types and not mlp_types:
        mlp_types = []
    return layer_types, mlp_types, mamba, gdn


# ---- canned shapes used by the benchmark configs ------------------------------------------

def qwen3_8b_config(**over: Any) -> ModelConfig:
    """Qwen3-8B geometry: 36 layers, hidden 4096, 32 q / 8 kv heads, d 128, I 12288, V 151936."""
    base = dict(model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                rms_norm_eps=1e-6, rope_theta=1e6, has_qk_norm=True, max_position_embeddings=40960)
    base.update(over)
    return ModelConfig(**base)


def qwen3_30b_a3b_config(**over: Any) -> ModelConfig:
    """Qwen3-30B-A3B geometry: 48 layers, hidden 2048, 32 q / 4 kv heads, 128 experts top-8, I_e 768."""
    base = dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                rms_norm_eps=1e-6, rope_theta=1e6, has_qk_norm=True, num_experts=128,
                num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True)
    base.update(over)
    return ModelConfig(**base)


def tiny_llama_config(**over: Any) -> ModelConfig:
    """The CPU plumbing-check model: 2 layers, hidden 256, 4 q / 2 kv heads, d 64, I 688, V 32000."""
    base = dict(model_type="llama", vocab_size=32000, hidden_size=256, intermediate_size=688,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                rms_norm_eps=1e-6, rope_theta=1e4, dtype="float32", max_position_embeddings=2048)
    base.update(over)
    return ModelConfig(**base)


def hybrid_nemotron_config(**over: Any) -> ModelConfig:
    """Hybrid benchmark shape: 52 layers, every 6th attention, every 4th Mamba layer a gated
    DeltaNet layer, the rest Mamba2; hidden 4096, MLP 16384."""
    n = over.pop("num_hidden_layers", 52)
    types: List[str] = []
    mamba_seen = 0
    for i in range(n):
        if (i + 1) % 6 == 0:
            types.append(LAYER_ATTENTION)
        else:
            mamba_seen += 1
            types.append(LAYER_GDN if mamba_seen % 4 == 0 else LAYER_MAMBA)
    base = dict(model_type="nemotron_h_hybrid", vocab_size=131072, hidden_size=4096, intermediate_size=16384,
                num_hidden_layers=n, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                rms_norm_eps=1e-5, rope_theta=1e4, layer_types=types, hidden_act="relu2",
                mamba=MambaConfig(), gdn=GdnConfig())
    base.update(over)
    return ModelConfig(**base)
