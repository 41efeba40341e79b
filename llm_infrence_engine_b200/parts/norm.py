"""RMS normalisation of rows of the 32-bit residual stream."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import INIT_NORM, VECTOR, Norm, ParamSpec, Source


class RMSNorm(Norm):
    """``y = weight * cast(x * rsqrt(mean(x^2) + eps))`` with the mean and the scaling in 32-bit.

    The reference reduces in 32-bit, casts to the model's dtype and multiplies by the weight there
    (src/miniserve/model.py:69-73). ``eps`` sits inside the square root, added to the mean.
    """

    graph_safe = True

    def __init__(self, dim: int, eps: float, weight_name: str):
        self.dim = dim
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((Source(self.weight_name, (self.dim,), INIT_NORM),), VECTOR)}

    def norm(self, ctx, residual):
        return ctx.K.add_rmsnorm(residual, None, self.weight, self.eps, ctx.dtype)

    def norm_rows(self, ctx, residual, rows):
        return ctx.K.rmsnorm_rows(residual, None, self.weight, self.eps, rows, ctx.dtype)
