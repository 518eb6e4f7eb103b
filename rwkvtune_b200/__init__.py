"""rwkvtune_b200: a Blackwell-native RWKV-7 training framework.

Public surface mirrors ``rwkvtune/__init__.py:24-93`` of the reference.  Heavy
sub-packages are imported lazily so that ``import rwkvtune_b200`` stays cheap.
"""
from __future__ import annotations

import importlib
from typing import Any

__version__ = "0.1.0"
__license__ = "Apache-2.0"
__author__ = "rwkvtune_b200 contributors"

_LAZY = {
    "RWKV7Model": "rwkvtune_b200.models", "RWKV7Config": "rwkvtune_b200.models",
    "RWKVConfig": "rwkvtune_b200.models", "GenerationConfig": "rwkvtune_b200.models",
    "AutoModel": "rwkvtune_b200.models",
    "get_tokenizer": "rwkvtune_b200.data.tokenizers", "TRIE_TOKENIZER": "rwkvtune_b200.data.tokenizers",
    "AutoTokenizer": "rwkvtune_b200.data.tokenizers", "RWKVTokenizer": "rwkvtune_b200.data.tokenizers",
    "PretrainConfig": "rwkvtune_b200.training", "PretrainTrainer": "rwkvtune_b200.training",
    "SFTConfig": "rwkvtune_b200.training", "SFTTrainer": "rwkvtune_b200.training",
    "GRPOConfig": "rwkvtune_b200.training", "GRPOTrainer": "rwkvtune_b200.training",
    "LoraConfig": "rwkvtune_b200.peft", "get_peft_model": "rwkvtune_b200.peft",
    "is_peft_model": "rwkvtune_b200.peft", "load_peft_model": "rwkvtune_b200.peft",
    "RWKV7_DEFAULT_TARGET_MODULES": "rwkvtune_b200.peft",
    "create_model_hub": "rwkvtune_b200.utils",
}
__all__ = ["__version__", "__author__", "__license__"] + sorted(_LAZY)


def __getattr__(name: str) -> Any:
    if name in _LAZY:
        return getattr(importlib.import_module(_LAZY[name]), name)
    raise AttributeError(f"module 'rwkvtune_b200' has no attribute {name!r}")
