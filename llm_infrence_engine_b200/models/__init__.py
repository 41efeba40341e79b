from . import qwen2  # noqa: F401  (registers the architecture)
from .registry import build_model_spec, known_architectures, lookup, parse_config, register_architecture
from .spec import LayerCall, ModelSpec, sequential

__all__ = ["build_model_spec", "known_architectures", "lookup", "parse_config", "register_architecture",
           "LayerCall", "ModelSpec", "sequential"]
