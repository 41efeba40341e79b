"""Trace replay: given token ids, step by step, through the engine's own step function; logits out.

Nothing is sampled. The steps come as JSON lines

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry brings the next tokens of one request; all entries of a step are one batch. ``want``
names the places among those tokens whose logits are written, ``end`` the requests that are over
after the step: their pages and slot go back to the pool, which is made for ``max_tokens`` tokens
only, so later requests get pages that earlier ones used. The model, the step function, the cache
manager and the kernels are the ones generation uses.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import Dict, IO, Iterable, Optional

import torch

from ..config.engine_config import EngineConfig
from .engine import build_runner
from .step import StepEntry

MAX_LIVE = 4      # requests that may be live at a time
ROUND_TO = 64     # every request's token count is rounded up to this when the pool is sized


class TraceReplayer:
    def __init__(self, model: str, dtype: str, max_tokens: int, device: str = "cuda:0", kernels=None, block_size: int = 16,
                 cuda_graphs: bool = False):
        if ROUND_TO % block_size:
            raise ValueError(f"block_size must divide {ROUND_TO}")
        pages = -(-max_tokens // block_size) + 1  # + the null page
        cfg = EngineConfig(dtype=dtype, device=device, block_size=block_size, num_blocks=pages, max_seqs=MAX_LIVE,
                           max_len=max(max_tokens, 1), max_num_batched_tokens=max(max_tokens, 1), cuda_graphs=cuda_graphs)
        self.spec, self.cache, self.runner = build_runner(model, cfg, kernels)
        self.lengths: Dict[str, int] = {}

    def step(self, record: dict) -> Optional[torch.Tensor]:
        """Run one line of the trace; returns float32 logits ``[wanted, vocab]`` on the host, or None."""
        entries = []
        for e in record.get("entries", []):
            rid = e["id"]
            tokens = list(e["tokens"])
            if rid not in self.lengths:
                self.cache.admit(rid)
                self.lengths[rid] = 0
            ctx = self.lengths[rid]
            self.cache.reserve(rid, ctx, ctx + len(tokens))
            entries.append(StepEntry(rid, tokens, ctx, list(e.get("want", []))))
        logits = self.runner.step(entries) if entries else None
        for e in entries:
            self.lengths[e.req] += len(e.tokens)
        for rid in record.get("end", []):
            if rid in self.lengths:
                self.cache.free(rid)
                del self.lengths[rid]
        return None if logits is None else logits.float().cpu()


def replay_stream(replayer: TraceReplayer, lines: Iterable[str], out_dir: Path, done: IO[str] = sys.stdout) -> None:
    out_dir.mkdir(parents=True, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = replayer.step(record)
        if logits is not None and logits.numel():
            logits.contiguous().numpy().astype("<f4").tofile(out_dir / f"{record['step']}.f32")
        done.write(f"done {record['step']}\n")
        done.flush()
