"""Grouped-query attention over a paged cache."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache.spec import PagedKVSpec
from .base import INIT_NORMAL, MATRIX, VECTOR, Mixer, ParamSpec, PositionEncoding, Source


class PagedAttention(Mixer):
    """``o_proj(softmax(q k^T * scale + causal mask) v)`` with ``num_heads`` query heads that share
    ``num_kv_heads`` key/value heads: query head ``h`` reads key/value head ``h // (num_heads // num_kv_heads)``
    (src/miniserve/model.py:121-152).

    The three projections are kept as one matrix ``[(num_heads + 2 num_kv_heads) * head_dim, hidden]``
    so a step multiplies once; the bias (if any), the rotation of q and k and the write of k and v
    into the request's pages are one kernel, or, in decode steps, the opening of the attention kernel itself
    (``qkv_attention`` of the kernels object decides). A token at position ``p`` sees keys ``0..p`` of its own
    request, or ``p - window + 1 .. p`` when ``window`` is set; the mask is never a tensor.
    """

    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, position: PositionEncoding,
                 prefix: str, bias: bool = True, window: Optional[int] = None, scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        self.hidden, self.num_heads, self.num_kv_heads, self.head_dim = hidden, num_heads, num_kv_heads, head_dim
        self.position = position
        self.prefix = prefix
        self.bias = bias
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)  # SDPA's default, model.py:143
        self.w_qkv: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        p, d, h = self.prefix, self.head_dim, self.hidden
        rows = (("q_proj", self.num_heads * d), ("k_proj", self.num_kv_heads * d), ("v_proj", self.num_kv_heads * d))
        out = {
            "w_qkv": ParamSpec(tuple(Source(f"{p}.{n}.weight", (r, h)) for n, r in rows), MATRIX),
            "w_o": ParamSpec((Source(f"{p}.o_proj.weight", (h, self.num_heads * d)),), MATRIX),
        }
        if self.bias:
            out["b_qkv"] = ParamSpec(tuple(Source(f"{p}.{n}.bias", (r,), INIT_NORMAL) for n, r in rows), VECTOR)
        return out

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        cos, sin = ctx.position_tables(self.position)
        attn = K.qkv_attention(h, self.w_qkv, self.b_qkv, cos, sin, ctx.slot_mapping[cache.group], cache.k, cache.v,
                               ctx.block_tables[cache.group], ctx.token_seq, ctx.positions, self.num_heads, self.num_kv_heads,
                               self.head_dim, ctx.page_size, self.scale, self.window or 0, ctx.max_context, batch=ctx,
                               write_kv=cache.write, out_dtype=ctx.dtype)
        K.linear(attn, self.w_o, add_to=residual)
