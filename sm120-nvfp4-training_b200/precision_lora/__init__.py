"""LoRA with preserved floating-point bases, NVFP4 re-packed bases, or packed NVFP4 checkpoint bases
(the public surface of the reference's src/precision_lora/__init__.py)."""
from .core import enable_lora, prepare_lora, lora_parameters, save_lora, load_lora, merge_lora, LoRALinear
from .graph import capture_lora_step
from .packed import PackedNVFP4Linear

__all__ = ["enable_lora", "prepare_lora", "lora_parameters", "save_lora", "load_lora", "merge_lora", "LoRALinear",
           "capture_lora_step", "PackedNVFP4Linear"]
