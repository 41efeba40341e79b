"""One layer: how norms, mixer and feed-forward are arranged around the residual stream."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .base import FeedForward, Mixer, Norm, Part


class PreNormBlock(Part):
    """``x += mixer(norm1(x)); x += ff(norm2(x))`` (src/miniserve/model.py:184-185).

    The residual stream ``x`` is 32-bit and is updated in place. The second addition is left to
    whoever normalises next (the following block, or the model's last norm), which does it in the
    same kernel as its norm: ``forward`` takes the addend still owed to ``x`` and returns the new one.
    """

    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ff: FeedForward):
        self.norm1, self.mixer, self.norm2, self.ff = norm1, mixer, norm2, ff

    def children(self) -> Sequence[Part]:
        return (self.norm1, self.mixer, self.norm2, self.ff)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, residual: torch.Tensor, delta: Optional[torch.Tensor], cache) -> torch.Tensor:
        h = self.norm1.add_norm(ctx, residual, delta)
        a = self.mixer.forward(ctx, h, cache)
        h = self.norm2.add_norm(ctx, residual, a)
        return self.ff.forward(ctx, h)
