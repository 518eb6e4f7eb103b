from .model_hub import create_model_hub

__all__ = ["create_model_hub"]
