"""What a mixer asks of the cache: pages of keys and values, or a state of fixed size, or nothing."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every cached token (or of the last ``window`` of them), kept in pages."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: all keys are kept; n: only keys p - n < j <= p are ever read


@dataclass(frozen=True)
class FixedStateSpec:
    """A per-request tensor of fixed shape that a mixer reads and writes in place (32-bit floats)."""

    shape: Tuple[int, ...]


NULL_PAGE = 0  # never handed out; block tables point at it where a request holds no page
