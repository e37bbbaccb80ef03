"""Post-training quantisation to the checkpoint layouts the runtime loads (NVFP4, INT4-AWQ).

Parity: ``tensorrt_edgellm/quantization/quantize.py:1309`` (``quantize_and_export``) and
``quantization_configs.py:226`` (``build_quant_config``).  The reference drives NVIDIA ModelOpt; this
module states the same arithmetic directly — max-calibrated per-tensor activation scales, block-16
E4M3-scaled E2M1 weights with an fp32 second-level scale, group-wise symmetric INT4 — and writes the
unified Hugging Face layout (``weight`` / ``weight_scale`` / ``weight_scale_2`` / ``input_scale`` plus
``hf_quant_config.json``)."""
from .quantize import build_quant_config, calibrate_input_scales, quantize_and_export

__all__ = ["build_quant_config", "calibrate_input_scales", "quantize_and_export"]
