"""Rotary position encoding: per-step cosine and sine tables from the tokens' absolute positions."""
from __future__ import annotations

import torch

from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
    """Angles ``position * theta^(-2j/d)`` for ``j < d/2``, in 32-bit; pairs are ``(j, j + d/2)``.

    The inverse frequencies are made the way the reference makes them (32-bit power and division,
    src/miniserve/model.py:83-85) so that both sides round alike; the reference then recomputes
    ``cos`` and ``sin`` on every forward (model.py:86-88), here the step does it once for all layers.
    """

    graph_safe = True

    def __init__(self, head_dim: int, theta: float):
        if head_dim % 2:
            raise ValueError(f"rotary head_dim must be even, got {head_dim}")
        self.head_dim = head_dim
        self.theta = float(theta)
        self._inv_freq = {}

    def key(self) -> tuple:
        return ("rotary", self.head_dim, self.theta)

    def inv_freq(self, device) -> torch.Tensor:
        dev = str(device)
        if dev not in self._inv_freq:
            f = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2).float() / self.head_dim))
            self._inv_freq[dev] = f.to(device)
        return self._inv_freq[dev]

    def tables(self, ctx):
        """(cos, sin), each ``[N, head_dim / 2]`` in 32-bit."""
        return ctx.K.rope_tables(ctx.positions, self.inv_freq(ctx.device))
