"""Dense gated feed-forward."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MATRIX, FeedForward, ParamSpec, Source

ACTIVATIONS = ("silu",)


class GatedMLP(FeedForward):
    """``down(act(gate(x)) * up(x))`` without biases (src/miniserve/model.py:164-165).

    ``gate`` and ``up`` are kept as one matrix ``[2 * intermediate, hidden]`` (gate rows first) so a
    step multiplies once; the activation and the product of the two halves are the epilogue of that product
    (prompt portions) or one kernel over its float32 sums (decode steps): ``gate_up_act`` of the kernels object decides.
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
        K.linear(K.gate_up_act(h, self.w_gate_up, ctx.dtype), self.w_down, add_to=residual)
