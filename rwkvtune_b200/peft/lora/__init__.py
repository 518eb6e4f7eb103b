from .layer import LoraLinear

__all__ = ["LoraLinear"]
