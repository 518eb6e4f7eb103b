"""Parameter-efficient fine-tuning (LoRA); public names of ``rwkvtune/peft/__init__.py:21-32``."""
from .config import RWKV7_DEFAULT_TARGET_MODULES, LoraConfig
from .lora.layer import LoraLinear
from .peft_model import get_peft_model, is_peft_model, load_peft_model

__all__ = ["LoraConfig", "LoraLinear", "RWKV7_DEFAULT_TARGET_MODULES", "get_peft_model", "is_peft_model", "load_peft_model"]
