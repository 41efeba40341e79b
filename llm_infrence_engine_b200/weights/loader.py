"""Weights from safetensors by tensor name, onto the device, into the parts of a model.

Every part names the checkpoint tensors it needs (``Part.params``). The loader checks the whole
checkpoint against that list before it reads a byte of data and raises ONE error that lists every
missing tensor, every unexpected one and every wrong shape. (The reference loads with
``strict=False`` and so ignores both silently, src/miniserve/loader.py:45.)

How a tensor is kept: matrices in the compute dtype (bfloat16 when serving, float32 in the 32-bit
path); vectors (norm weights, biases) always in float32, so one stored in 32-bit stays so and one
stored in bfloat16 is widened exactly; integer tables as int32. Projections that a part multiplies
together are joined along their output rows here, once.
"""
from __future__ import annotations

import warnings
from pathlib import Path
from typing import Dict, List, Tuple

import torch

from ..models.spec import ModelSpec
from ..parts.base import MATRIX, TABLE, VECTOR, ParamSpec, Part
from .safetensors_io import SafetensorsFile

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightsError(ValueError):
    """The checkpoint does not fit the model; the message lists everything that is wrong."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected, self.wrong_shape, self.wrong_dtype = missing, unexpected, wrong_shape, wrong_dtype
        lines = [f"weights in {folder} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, got, want in wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, the model needs {list(want)}")
        for name, got, want in wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {got}, the model needs {want}")
        super().__init__("\n".join(lines))


def _target_dtype(kind: str, compute: torch.dtype) -> torch.dtype:
    return {MATRIX: compute, VECTOR: torch.float32, TABLE: torch.int32}[kind]


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[Tuple[int, ...], str, bool]]:
    """Checkpoint name -> (shape, kind, optional) over all parts of the model."""
    out: Dict[str, Tuple[Tuple[int, ...], str, bool]] = {}
    for part in spec.parts():
        for p in part.params().values():
            for s in p.sources:
                if s.name in out and out[s.name][0] != tuple(s.shape):
                    raise ValueError(f"two parts ask for '{s.name}' with different shapes")
                out[s.name] = (tuple(s.shape), p.kind, s.optional)
    return out


def load_weights(spec: ModelSpec, folder: str | Path, dtype: torch.dtype, device) -> int:
    """Fill every part of ``spec`` from the ``*.safetensors`` files of ``folder``; returns the bytes put on the device."""
    folder = Path(folder)
    paths = sorted(folder.glob("*.safetensors"))  # sorted, later files win, as src/miniserve/loader.py:41-43
    if not paths:
        raise FileNotFoundError(f"no .safetensors file in {folder}")
    files = [SafetensorsFile(p) for p in paths]
    try:
        where: Dict[str, SafetensorsFile] = {}
        for f in files:
            for name in f.names():
                where[name] = f
        want = expected_tensors(spec)
        ignored = set()
        for part in spec.parts():
            ignored.update(getattr(part, "ignored_names", lambda: ())())

        missing = [n for n, (_, _, opt) in want.items() if n not in where and not opt]
        unexpected = [n for n in where if n not in want and n not in ignored]
        wrong_shape, wrong_dtype = [], []
        for name, (shape, kind, _) in want.items():
            if name not in where:
                continue
            got_dtype, got_shape = where[name].info(name)
            if tuple(got_shape) != tuple(shape):
                wrong_shape.append((name, got_shape, shape))
            if kind == TABLE and got_dtype not in _INTS:
                wrong_dtype.append((name, got_dtype, "an integer type"))
            if kind != TABLE and got_dtype not in _FLOATS:
                wrong_dtype.append((name, got_dtype, "a floating type"))
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightsError(folder, sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)

        # A tensor that is present but stands aside for another (the output head of a tied checkpoint) should be that
        # other tensor; the reference re-ties without looking (src/miniserve/loader.py:46-47). Here a difference is said.
        for part in spec.parts():
            for aside, used in getattr(part, "aliases", lambda: {})().items():
                if aside in where and used in where:
                    a, b = where[aside].tensor(aside), where[used].tensor(used)
                    if a.shape != b.shape or not torch.equal(a, b):
                        warnings.warn(f"{folder}: '{aside}' differs from '{used}', which the configuration ties it to; "
                                      f"'{aside}' is not used", stacklevel=2)

        total = 0
        for part in spec.parts():
            bound = {}
            for local, p in part.params().items():
                target = _target_dtype(p.kind, dtype)
                pieces = [where[s.name].tensor(s.name).to(target) for s in p.sources if s.name in where]
                t = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
                bound[local] = t.contiguous().to(device)
                total += t.numel() * t.element_size()
            part.bind(bound)
        return total
    finally:
        for f in files:
            f.close()
