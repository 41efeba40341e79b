"""A request and the record of one step, with the reference's field names where it has them
(src/miniserve/engine.py:32-91)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple


@dataclass(eq=False)  # a request is itself, not its field values: lists of requests are searched by identity
class Request:
    prompt_ids: List[int]
    max_new_tokens: int = 64
    eos_ids: Tuple[int, ...] = ()
    temperature: float = 0.0     # <= 0: greedy
    top_k: int = 0               # 0: off
    top_p: float = 1.0           # 1: off
    seed: Optional[int] = None   # None: the engine's seed plus the request's id
    ignore_eos: bool = False     # keep generating through stop tokens (src/miniserve/server.py:56,292)

    # --- filled in by the engine ---
    id: int = -1
    state: str = "waiting"       # waiting -> running -> finished (a preempted request waits again, keeping its output)
    output_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None  # "stop" | "length" | "abort"
    cancelled: bool = False
    num_computed: int = 0        # tokens of prompt + output whose keys and values are in the cache
    in_flight: int = 0           # tokens chosen on the device that the host has not read yet (pipelined engine): 0 or 1
    preemptions: int = 0
    admit_seq: int = 0           # admission order; the youngest is preempted first
    arrival_time: float = 0.0
    admitted_time: Optional[float] = None
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    token_times: List[float] = field(default_factory=list)

    @property
    def all_ids(self) -> List[int]:
        return self.prompt_ids + self.output_ids

    @property
    def num_tokens(self) -> int:
        """Tokens so far: prompt plus output, the one still on the device included."""
        return len(self.prompt_ids) + len(self.output_ids) + self.in_flight

    def tokens(self, start: int, stop: int) -> List[int]:
        """``all_ids[start:stop]`` without joining the two lists."""
        p = len(self.prompt_ids)
        if stop <= p:
            return self.prompt_ids[start:stop]
        if start >= p:
            return self.output_ids[start - p:stop - p]
        return self.prompt_ids[start:] + self.output_ids[:stop - p]

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival_time

    @property
    def e2e(self) -> Optional[float]:
        return None if self.finish_time is None else self.finish_time - self.arrival_time


@dataclass
class StepRecord:
    n_prefill: int            # requests admitted in this step
    decode_batch: int         # requests that brought one decoded token
    useful_rows: int          # tokens emitted
    duration: float
    n_preempted: int = 0
    num_tokens: int = 0       # rows of the step's batch
    num_prefill_tokens: int = 0


@dataclass
class GenerationResult:
    """What ``generate`` returns for one prompt (src/miniserve/generate.py:19-37)."""

    token_ids: List[int]
    prompt_len: int
    ttft: float
    total_time: float
    step_times: List[float] = field(default_factory=list)
    finish_reason: str = "length"
    cache_bytes: int = 0

    @property
    def decode_tps(self) -> float:
        t = sum(self.step_times)
        return len(self.step_times) / t if t > 0 else 0.0
