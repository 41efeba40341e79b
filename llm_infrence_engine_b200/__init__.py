"""A small, whole inference engine for the dense Qwen2 decoder on one B200."""
from .config import ConfigError, EngineConfig, Qwen2Config

__all__ = ["ConfigError", "EngineConfig", "Qwen2Config"]
__version__ = "0.1.0"
