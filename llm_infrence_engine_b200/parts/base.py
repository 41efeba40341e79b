"""Interfaces of the parts a model is put together from.

A part owns its sizes and constants (constructor arguments), names the checkpoint tensors it
needs, and runs on a flat batch of tokens. It never learns which model it is in: everything about
the running step reaches it through a ``StepContext``.

Kinds of part and what each must provide:

``Norm``              ``norm(ctx, residual) -> h``: the rows of the 32-bit residual stream, normalised, in the
                      compute dtype; ``norm_rows(ctx, residual, rows)`` the same for chosen rows only.
``PositionEncoding``  ``tables(ctx) -> object``: whatever its mixers need for the step's positions;
                      the context computes it once per step and shares it between layers.
``Mixer``             ``cache_spec()`` (pages, fixed state or None) and ``forward(ctx, h, cache, residual)``:
                      reads and writes only its ``cache`` and ADDS its ``[N, hidden]`` result into ``residual``.
``FeedForward``       ``forward(ctx, h, residual)``: adds its result into ``residual``.
``Block``             the arrangement of the above in one layer: ``forward(ctx, residual, cache)``.

Every part lists its tensors with ``params()``; the loader fills them and calls ``bind``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

# How a checkpoint tensor is kept on the device.
MATRIX = "matrix"  # compute dtype (bfloat16 when serving, float32 in the 32-bit path)
VECTOR = "vector"  # always float32: small, and a tensor stored in 32-bit stays so
TABLE = "table"    # integers, kept as int32

# How the random-weights mode draws a checkpoint tensor.
INIT_NORMAL = "normal"      # N(0, 0.02): matrices, embeddings and biases
INIT_NORM = "norm_weight"   # 1 + U(-0.1, 0.1): weights of norms


@dataclass(frozen=True)
class Source:
    """One tensor of the checkpoint: its name, its shape there and how random mode draws it."""

    name: str
    shape: Tuple[int, ...]
    init: str = INIT_NORMAL
    optional: bool = False  # may be absent (for instance the output head of a tied checkpoint)


@dataclass(frozen=True)
class ParamSpec:
    """One device tensor of a part: one checkpoint tensor, or several joined along dim 0."""

    sources: Tuple[Source, ...]
    kind: str = MATRIX

    @property
    def shape(self) -> Tuple[int, ...]:
        first = self.sources[0].shape
        return (sum(s.shape[0] for s in self.sources),) + tuple(first[1:])


class Part:
    """Base of every part: named tensors in, ``bind`` once, then ``forward`` every step."""

    # True if ``forward`` only launches kernels on the current stream and reads nothing of the step on the
    # host (no host lists of the context, no synchronisation): such a part can be captured in a CUDA graph.
    graph_safe = False

    def params(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for name, t in tensors.items():
            setattr(self, name, t)

    def children(self) -> Sequence["Part"]:
        return ()

    def weight_bytes(self) -> int:
        """Bytes of this part's own tensors that one step reads (children not included)."""
        n = 0
        for name in self.params():
            t = getattr(self, name, None)
            if t is not None:
                n += t.numel() * t.element_size()
        return n


class Norm(Part):
    def norm(self, ctx, residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def norm_rows(self, ctx, residual: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Normalise only ``residual[rows]``."""
        raise NotImplementedError


class PositionEncoding(Part):
    def key(self) -> tuple:
        """Two encodings with equal keys give equal tables, which a step then computes once."""
        raise NotImplementedError

    def tables(self, ctx):
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, ctx, h: torch.Tensor, cache, residual: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


def walk(part: Part) -> List[Part]:
    """The part and everything under it, parents first."""
    out = [part]
    for c in part.children():
        out.extend(walk(c))
    return out
