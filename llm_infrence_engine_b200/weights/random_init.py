"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference has no such mode (its tests download the real checkpoint, tests/conftest.py:26-36).
Tensors are drawn on the CPU in 32-bit, one after the other in the order in which the model's
parts name them, from one generator: the same configuration and seed always give the same folder.
Matrices, embeddings and biases are N(0, std); weights of norms are 1 + U(-0.1, 0.1).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict, Mapping

import torch

from ..models.registry import build_model_spec
from ..parts.base import INIT_NORM, INIT_NORMAL
from .safetensors_io import write_safetensors

_STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def random_tensors(config_json: Mapping[str, Any], seed: int, std: float = 0.02) -> Dict[str, torch.Tensor]:
    spec = build_model_spec(config_json)
    gen = torch.Generator().manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for part in spec.parts():
        for p in part.params().values():
            for s in p.sources:
                if s.name in out:
                    continue
                if s.init == INIT_NORM:
                    t = 1.0 + (torch.rand(s.shape, generator=gen) * 0.2 - 0.1)
                elif s.init == INIT_NORMAL:
                    t = torch.randn(s.shape, generator=gen) * std
                else:
                    raise ValueError(f"tensor '{s.name}' asks for unknown initialisation '{s.init}'")
                out[s.name] = t
    return out


def write_random_model(config_json: Mapping[str, Any], folder: str | Path, seed: int = 0, store_dtype: str = "float32",
                       std: float = 0.02) -> Path:
    """Write ``folder/config.json`` and ``folder/model.safetensors``; returns the folder."""
    if store_dtype not in _STORE:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE)}")
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config_json, seed, std)
    write_safetensors(folder / "model.safetensors", {k: v.to(_STORE[store_dtype]) for k, v in tensors.items()})
    cfg = dict(config_json)
    cfg["torch_dtype"] = store_dtype
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    return folder
