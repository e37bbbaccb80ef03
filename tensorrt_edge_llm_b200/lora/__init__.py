"""LoRA adapters: processing into the runtime layout and merging into a checkpoint.

Parity: ``tensorrt_edgellm/lora/lora.py`` (insert / process / merge) and the runtime contract of
``cpp/runtime/state/loraManager.{h,cpp}`` (named adapters, tensors ``lora_A_<module>`` ``[r, in]`` and
``lora_B_<module>`` ``[out, r]`` with the ``alpha / r`` scale folded into B)."""
from .lora import lora_target_modules, merge_lora, process_lora_weights
from .runtime import LoraLinear, LoraManager

__all__ = ["lora_target_modules", "merge_lora", "process_lora_weights", "LoraLinear", "LoraManager"]
