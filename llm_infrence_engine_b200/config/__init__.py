from .engine_config import EngineConfig
from .model_config import ConfigError, Qwen2Config, architecture_name, read_config_json

__all__ = ["ConfigError", "EngineConfig", "Qwen2Config", "architecture_name", "read_config_json"]
