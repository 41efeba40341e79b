"""One layer: how norms, mixer and feed-forward are arranged around the residual stream."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .base import FeedForward, Mixer, Norm, Part


class PreNormBlock(Part):
    """``x += mixer(norm1(x)); x += ff(norm2(x))`` (src/miniserve/model.py:184-185).

    The residual stream ``x`` is 32-bit and is updated in place: the mixer and the feed-forward are handed
    ``x`` and add their result into it themselves, which lets their last matrix product do the addition
    in its own epilogue instead of a kernel of its own.
    """

    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ff: FeedForward):
        self.norm1, self.mixer, self.norm2, self.ff = norm1, mixer, norm2, ff

    def children(self) -> Sequence[Part]:
        return (self.norm1, self.mixer, self.norm2, self.ff)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, residual: torch.Tensor, cache) -> None:
        self.mixer.forward(ctx, self.norm1.norm(ctx, residual), cache, residual)
        self.ff.forward(ctx, self.norm2.norm(ctx, residual), residual)
