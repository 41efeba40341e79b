"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import MATRIX, ParamSpec, Part, Source


class TokenEmbedding(Part):
    """``x = table[token]`` with no scaling (src/miniserve/model.py:229), widened into the 32-bit residual stream."""

    graph_safe = True

    def __init__(self, vocab: int, hidden: int, name: str):
        self.vocab, self.hidden, self.name = vocab, hidden, name
        self.table: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        return {"table": ParamSpec((Source(self.name, (self.vocab, self.hidden)),), MATRIX)}

    def forward(self, ctx) -> torch.Tensor:
        return ctx.K.embed(ctx.token_ids, self.table)


class OutputHead(Part):
    """``logits = h W^T`` without bias, in 32-bit. ``tied_to`` makes ``W`` the embedding's own table
    (src/miniserve/model.py:204-206); a tensor of the head's name in the checkpoint is then not needed."""

    graph_safe = True

    def __init__(self, vocab: int, hidden: int, name: str, tied_to: Optional[TokenEmbedding] = None):
        self.vocab, self.hidden, self.name, self.tied_to = vocab, hidden, name, tied_to
        self.weight: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        if self.tied_to is not None:
            return {}
        return {"weight": ParamSpec((Source(self.name, (self.vocab, self.hidden)),), MATRIX)}

    def ignored_names(self):
        """Checkpoint names that may be present without being read."""
        return (self.name,) if self.tied_to is not None else ()

    def aliases(self) -> Dict[str, str]:
        """Ignored checkpoint name -> the tensor that stands in for it; the loader warns when the two differ."""
        return {self.name: self.tied_to.name} if self.tied_to is not None else {}

    def matrix(self) -> torch.Tensor:
        return self.tied_to.table if self.tied_to is not None else self.weight

    def forward(self, ctx, h: torch.Tensor) -> torch.Tensor:
        return ctx.K.linear(h, self.matrix(), out_dtype=torch.float32)
