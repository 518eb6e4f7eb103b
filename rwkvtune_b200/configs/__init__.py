from .model_loader import ModelConfig, list_available_models, load_model_config, print_model_info

__all__ = ["ModelConfig", "list_available_models", "load_model_config", "print_model_info"]
