from .model_config import ModelConfig, Qwen3Config
from .runtime_config import RuntimeConfig

__all__ = ["ModelConfig", "Qwen3Config", "RuntimeConfig"]
