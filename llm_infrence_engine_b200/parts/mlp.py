"""Dense gated feed-forward."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MATRIX, FeedForward, ParamSpec, Source

ACTIVATIONS = ("silu",)


class GatedMLP(FeedForward):
    """``down(act(gate(x)) * up(x))`` without biases (src/miniserve/model.py:164-165).

    ``gate`` and ``up`` are kept as one matrix ``[2 * intermediate, hidden]`` (gate rows first) so a
    step multiplies once; the activation and the product are one kernel over its output.
    """

    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, prefix: str, activation: str = "silu"):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not one of {ACTIVATIONS}")
        self.hidden, self.intermediate, self.prefix, self.activation = hidden, intermediate, prefix, activation
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        p, h, i = self.prefix, self.hidden, self.intermediate
        return {
            "w_gate_up": ParamSpec((Source(f"{p}.gate_proj.weight", (i, h)), Source(f"{p}.up_proj.weight", (i, h))), MATRIX),
            "w_down": ParamSpec((Source(f"{p}.down_proj.weight", (h, i)),), MATRIX),
        }

    def forward(self, ctx, h, residual):
        K = ctx.K
        gu = K.linear(h, self.w_gate_up, transient=True)
        K.linear(K.silu_mul(gu, ctx.dtype), self.w_down, add_to=residual)
