"""Settings of the engine around a model: cache pool, batch limits, precision.

The names follow the reference's constructor arguments and command line where it has them
(src/miniserve/paged_engine.py:25-36, src/miniserve/server.py:435-448): ``block_size`` (16),
``num_blocks``, ``max_seqs`` (32), ``max_len``. ``max_num_batched_tokens`` is the token budget of
one step, which the reference does not have because it never cuts a prompt.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPES = ("bfloat16", "float32")


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"          # "bfloat16": serving kernels; "float32": everything in true 32-bit
    device: str = "cuda:0"
    block_size: int = 16             # tokens in a cache page
    num_blocks: Optional[int] = None  # pages in each group's pool, the null page included; None: from max_seqs * max_len
    max_seqs: int = 32               # requests that may hold cache at a time (also the number of state slots)
    max_len: int = 1024              # most tokens (prompt + generated) one request may reach
    max_num_batched_tokens: int = 2048  # token budget of one step
    cuda_graphs: bool = False        # replay decode-only steps from captured graphs
    pipeline: bool = False           # launch a step before the host has read the tokens of the step before it
    prefix_cache: bool = False       # requests take over cached pages that hold their leading tokens (one unwindowed group, no state)
    seed: int = 0                    # engine seed for requests that bring none

    def validate(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        if self.block_size <= 0:
            raise ValueError("block_size must be positive")
        if self.max_seqs <= 0 or self.max_len <= 0 or self.max_num_batched_tokens <= 0:
            raise ValueError("max_seqs, max_len and max_num_batched_tokens must be positive")
        if self.num_blocks is not None and self.num_blocks < 2:
            raise ValueError("num_blocks must be at least 2 (page 0 is the null page)")

    def pool_blocks(self) -> int:
        """Pages per pool: what was asked for, else room for max_seqs requests of max_len (server.py:145)."""
        if self.num_blocks is not None:
            return self.num_blocks
        per_seq = -(-self.max_len // self.block_size)
        return self.max_seqs * per_seq + 1
