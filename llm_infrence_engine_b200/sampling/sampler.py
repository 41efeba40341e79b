"""From logits to the next token of every row: greedy, temperature, top-k, top-p.

The distribution is the reference's (src/miniserve/sampler.py:12-41): logits / temperature; keep
the logits that are at least the k-th largest; in descending order drop a token once the mass
before it reaches top_p (the first is always kept); softmax. ``temperature <= 0`` is the argmax.
All of it runs on the device, one kernel for the rows of a step, and one copy brings the chosen
ids to the host (the reference already batches its greedy rows that way, src/miniserve/engine.py:260-277).

The draw differs from the reference's on purpose: ``torch.multinomial`` with a per-request
``torch.Generator`` (sampler.py:54-55) cannot be reproduced inside a kernel, so a row's uniform
number comes from a counter-based hash of (its seed, the index of the token being drawn) and the
token is the first one, in index order, whose running mass exceeds it. A request therefore draws
the same tokens whatever else is in the batch and after a preemption.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

_MASK = (1 << 64) - 1


def uniform_from(seed: int, counter: int) -> float:
    """The number in [0, 1) that the sampling kernel uses for (seed, counter): two rounds of the
    splitmix64 finaliser over their combination, top 24 bits."""
    z = (seed * 0x9E3779B97F4A7C15 + (counter + 1) * 0xBF58476D1CE4E5B9) & _MASK
    for _ in range(2):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must be 0 (off) or positive")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")


class Sampler:
    def __init__(self, kernels):
        self.K = kernels

    def sample_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int],
                      greedy_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits ``[M, vocab]`` float32 on the device -> M token ids (int32) still on the device. ``greedy_tokens``: the
        rows' argmax if the step already made it."""
        if logits.shape[0] != len(params):
            raise ValueError("one SamplingParams per row of logits is needed")
        if all(p.temperature <= 0.0 for p in params):
            if greedy_tokens is not None and greedy_tokens.shape[0] == logits.shape[0]:
                return greedy_tokens
            return self.K.argmax(logits)
        dev = logits.device
        t = torch.tensor([p.temperature for p in params], dtype=torch.float32).to(dev)
        k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(dev)
        pp = torch.tensor([p.top_p for p in params], dtype=torch.float32).to(dev)
        u = torch.tensor([uniform_from(p.seed, c) for p, c in zip(params, counters)], dtype=torch.float32).to(dev)
        return self.K.sample(logits, t, k, pp, u)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int],
               greedy_tokens: Optional[torch.Tensor] = None) -> List[int]:
        """The same, read back: M token ids on the host."""
        return self.sample_device(logits, params, counters, greedy_tokens).tolist()
