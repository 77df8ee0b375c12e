"""LoRA entry points re-exported from precision_lora, as in the reference's src/nvfp4_training/lora.py."""
from precision_lora.core import (enable_lora, prepare_lora, lora_parameters, save_lora, load_lora, merge_lora, LoRALinear,
                                 _LoRAFunction, _FrozenFP4)
from precision_lora.packed import PackedNVFP4Linear
from precision_lora.graph import LoRAStep, capture_lora_step
