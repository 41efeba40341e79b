"""Typed model configurations, read from the architecture's own ``config.json`` keys.

A configuration class knows the keys of one architecture, their defaults and the combinations that
make no sense. It holds every size and constant of the model; code below it takes them as
parameters and never writes one down itself.

The reference reads nine keys into ``ModelConfig`` (src/miniserve/model.py:26-58) and derives
``head_dim``; the class here reads the same keys with the same defaults and adds the ones the
checkpoint format carries but the reference ignores (explicit ``head_dim``, the sliding window
triple, ``attention_bias``, ``hidden_act``, ``max_position_embeddings``).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, fields
from pathlib import Path
from typing import Any, Mapping, Optional


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong kind, or asks for an impossible model."""


def _need(d: Mapping[str, Any], key: str, kind):
    if key not in d:
        raise ConfigError(f"config.json has no '{key}'")
    v = d[key]
    if kind is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if (isinstance(v, bool) and kind is not bool) or not isinstance(v, kind):
        raise ConfigError(f"config.json: '{key}' must be {kind.__name__}, got {v!r}")
    return v


def _refuse_unread_arithmetic(d: Mapping[str, Any]) -> None:
    """Keys that change the model's arithmetic and that this engine does not carry out: a checkpoint that sets one of
    them would give wrong logits without a word (the reference reads none of them, src/miniserve/model.py:42-58, and
    is silent). A key that is absent, null or at its neutral value is fine."""
    nested = d.get("rope_parameters") if isinstance(d.get("rope_parameters"), Mapping) else {}
    scaling = d.get("rope_scaling")
    if scaling is None and nested.get("rope_type") not in (None, "default"):
        scaling = {k: v for k, v in nested.items() if k != "rope_theta"}
    if isinstance(scaling, Mapping) and (scaling.get("rope_type") or scaling.get("type")) == "default":
        scaling = None
    if scaling is not None:
        raise ConfigError(f"config.json: 'rope_scaling' is {scaling!r}; scaled rotary positions are not built here "
                          "(only plain rotary positions with 'rope_theta')")
    prf = d.get("partial_rotary_factor", nested.get("partial_rotary_factor"))
    if prf is not None and float(prf) != 1.0:
        raise ConfigError(f"config.json: 'partial_rotary_factor' is {prf!r}; only whole heads are rotated here (1.0)")
    drop = d.get("attention_dropout")
    if drop is not None and float(drop) != 0.0:
        raise ConfigError(f"config.json: 'attention_dropout' is {drop!r}; an inference engine has none (0.0)")
    if d.get("mlp_bias"):
        raise ConfigError("config.json: 'mlp_bias' is true; the feed-forward of Qwen2 has no biases")


@dataclass(frozen=True)
class Qwen2Config:
    """The dense Qwen2 decoder: GQA attention with QKV bias, rotary positions, RMSNorm, SwiGLU."""

    architecture = "Qwen2ForCausalLM"

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    attention_bias: bool = True
    hidden_act: str = "silu"
    max_position_embeddings: int = 32768
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        _refuse_unread_arithmetic(d)
        heads = _need(d, "num_attention_heads", int)
        hidden = _need(d, "hidden_size", int)
        rope = d.get("rope_theta")
        if rope is None:  # newer checkpoints nest it (src/miniserve/model.py:45-47)
            rope = (d.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if heads <= 0 or hidden % heads:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads  # src/miniserve/model.py:38-40
        cfg = cls(
            vocab_size=_need(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size", int),
            num_hidden_layers=_need(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=_need(d, "num_key_value_heads", int),
            head_dim=int(head_dim),
            rms_norm_eps=_need(d, "rms_norm_eps", float),
            rope_theta=float(rope),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", True)),
            hidden_act=str(d.get("hidden_act", "silu")),
            max_position_embeddings=int(d.get("max_position_embeddings", 32768)),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=d.get("sliding_window"),
            max_window_layers=int(d.get("max_window_layers", 0) or 0),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act '{self.hidden_act}' is not known to Qwen2 (only 'silu')")
        if self.use_sliding_window and (not isinstance(self.sliding_window, int) or self.sliding_window <= 0):
            raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")

    # ------------------------------------------------------------------ derived
    def layer_window(self, layer: int) -> Optional[int]:
        """Keys a layer may look back over (itself included), or None for all of them."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return None

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen2"
        return d


def read_config_json(folder: str | Path) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d


def architecture_name(d: Mapping[str, Any]) -> str:
    arch = d.get("architectures")
    if not isinstance(arch, (list, tuple)) or not arch or not isinstance(arch[0], str):
        raise ConfigError("config.json has no 'architectures' list naming the model class")
    return arch[0]


def config_field_names(cls) -> list[str]:
    return [f.name for f in fields(cls)]
