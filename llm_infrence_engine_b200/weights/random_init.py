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
from .safetensors_io import write_safetensors_stream

_STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _sources(config_json: Mapping[str, Any]):
    """Every checkpoint tensor of the model once, in the order in which the model's parts name them."""
    spec = build_model_spec(config_json)
    seen = set()
    for part in spec.parts():
        for p in part.params().values():
            for s in p.sources:
                if s.name not in seen:
                    seen.add(s.name)
                    yield s


def _draw(s, gen: torch.Generator, std: float) -> torch.Tensor:
    if s.init == INIT_NORM:
        return 1.0 + (torch.rand(s.shape, generator=gen) * 0.2 - 0.1)
    if s.init == INIT_NORMAL:
        return torch.randn(s.shape, generator=gen) * std
    raise ValueError(f"tensor '{s.name}' asks for unknown initialisation '{s.init}'")


def random_tensors(config_json: Mapping[str, Any], seed: int, std: float = 0.02) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(int(seed))
    return {s.name: _draw(s, gen, std) for s in _sources(config_json)}


def write_random_model(config_json: Mapping[str, Any], folder: str | Path, seed: int = 0, store_dtype: str = "float32",
                       std: float = 0.02) -> Path:
    """Write ``folder/config.json`` and ``folder/model.safetensors``; returns the folder. Tensors are drawn and written one
    after the other (the same numbers as ``random_tensors`` gives), so a model of many gigabytes needs no more host memory
    than its largest tensor."""
    if store_dtype not in _STORE:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE)}")
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    dtype = _STORE[store_dtype]
    sources = list(_sources(config_json))
    by_name = {s.name: s for s in sources}
    gen = torch.Generator().manual_seed(int(seed))
    write_safetensors_stream(folder / "model.safetensors", [(s.name, dtype, tuple(s.shape)) for s in sources],
                             lambda name: _draw(by_name[name], gen, std).to(dtype))
    cfg = dict(config_json)
    cfg["torch_dtype"] = store_dtype
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    return folder
