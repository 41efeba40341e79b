"""A model as data: its parts and the order in which its layers run."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Sequence

from ..parts.base import Norm, Part, walk
from ..parts.embedding import OutputHead, TokenEmbedding


@dataclass(frozen=True)
class LayerCall:
    """One entry of the running order: which layer runs and which cache entry it uses.

    A layer may be named by several calls (its weights run again), each with a cache entry of its
    own; and a call with ``write=False`` reads a cache entry that an earlier call filled instead
    of keeping one itself.
    """

    layer: int
    cache: int
    write: bool = True


@dataclass
class ModelSpec:
    config: Any
    embedding: TokenEmbedding
    layers: List[Part]              # each has forward(ctx, residual, cache) and cache_spec()
    schedule: List[LayerCall]
    final_norm: Norm
    head: OutputHead

    def parts(self) -> List[Part]:
        out: List[Part] = []
        for top in [self.embedding, *self.layers, self.final_norm, self.head]:
            out.extend(walk(top))
        return out

    def cache_specs(self) -> list:
        """The spec of every cache entry, taken from the call that writes it."""
        n = 1 + max((c.cache for c in self.schedule), default=-1)
        specs: list = [None] * n
        written = [False] * n
        for call in self.schedule:
            spec = self.layers[call.layer].cache_spec()
            if call.write:
                if written[call.cache]:
                    raise ValueError(f"cache entry {call.cache} is written by two calls of the running order")
                specs[call.cache], written[call.cache] = spec, True
        for call in self.schedule:
            if not call.write:
                if not written[call.cache]:
                    raise ValueError(f"cache entry {call.cache} is read but no call writes it")
                if self.layers[call.layer].cache_spec() != specs[call.cache]:
                    raise ValueError(f"layer {call.layer} reads cache entry {call.cache} of another shape")
        return specs

    def vocab_size(self) -> int:
        return self.head.vocab


def sequential(num_layers: int) -> List[LayerCall]:
    """Layers 0..n-1 once each, every one with its own cache entry."""
    return [LayerCall(i, i) for i in range(num_layers)]
