from .configuration import GenerationConfig, RWKVConfig
from .auto_model import AutoModel
from .generation_mixin import GenerationMixin
from .rwkv7 import RWKV7Config, RWKV7Model

__all__ = ["RWKVConfig", "GenerationConfig", "AutoModel", "RWKV7Model", "RWKV7Config", "GenerationMixin"]
