"""Graph replay of a LoRA update, re-exported as in the reference's src/nvfp4_training/lora_graph.py."""
from precision_lora.graph import LoRAStep, capture_lora_step
