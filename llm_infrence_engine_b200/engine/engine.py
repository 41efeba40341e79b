"""The engine: a model folder in, generated tokens out, with the reference's calls where it has them.

``Engine.add_request`` / ``step`` / ``has_work`` / ``run_until_idle`` / ``cancel`` / ``stats`` follow
src/miniserve/engine.py:143-205 and src/miniserve/paged_engine.py:57-80; ``Engine.generate`` and the
module-level ``generate`` take the options of src/miniserve/generate.py:85-96 and return its
``GenerationResult``. Below the surface nothing is the reference's: one step function runs prompt
portions and decoded tokens together, and the pages, slots and decisions are in
``cache.CacheManager`` and ``engine.Scheduler``.
"""
from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Callable, List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..config.model_config import read_config_json
from ..models.registry import build_model_spec
from ..models.spec import ModelSpec
from ..sampling.sampler import Sampler, SamplingParams
from ..weights.loader import load_weights
from .request import GenerationResult, Request, StepRecord
from .scheduler import Scheduler, StepPlan
from .step import ModelRunner, StepEntry, group_layout

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def build_runner(folder: Union[str, Path], config: EngineConfig, kernels=None):
    """config.json -> registry -> parts -> weights -> cache; returns (spec, cache manager, runner)."""
    config.validate()
    if kernels is None:
        from ..csrc import get_kernels  # compiles at its first call; raises if there is no CUDA device or compiler

        kernels = get_kernels()
    spec = build_model_spec(read_config_json(folder))
    dtype = _TORCH_DTYPE[config.dtype]
    load_weights(spec, folder, dtype, config.device)
    groups, of_entry = group_layout(spec.cache_specs())
    num_pages = config.pool_blocks()
    stateless = all(e is not None for e in of_entry)  # every cache entry is paged: no fixed-size state to snapshot
    cache = CacheManager(groups, num_pages, config.block_size, config.max_seqs, prefix_sharing=config.prefix_cache and stateless)
    runner = ModelRunner(spec, kernels, cache, of_entry, dtype, config.device, num_pages, config.block_size, config.max_seqs,
                         config.max_len, config.cuda_graphs)
    return spec, cache, runner


class Engine:
    def __init__(self, model: Union[str, Path], config: Optional[EngineConfig] = None, kernels=None,
                 on_token: Optional[Callable[[Request, int], None]] = None,
                 on_finish: Optional[Callable[[Request], None]] = None,
                 clock: Callable[[], float] = time.perf_counter, **overrides):
        self.config = config or EngineConfig()
        for k, v in overrides.items():
            if not hasattr(self.config, k):
                raise TypeError(f"EngineConfig has no option '{k}'")
            setattr(self.config, k, v)
        self.spec, self.cache, self.runner = build_runner(model, self.config, kernels)
        self.scheduler = Scheduler(self.cache, self.config.max_seqs, self.config.max_len, self.config.max_num_batched_tokens)
        self.sampler = Sampler(self.runner.K)
        self.on_token, self.on_finish, self.clock = on_token, on_finish, clock
        self.finished: List[Request] = []
        self.steps: List[StepRecord] = []
        self.peak_running = 0
        self.peak_pages_in_use = 0
        self.prefill_tokens_computed = 0
        self._pipeline = bool(self.config.pipeline) and torch.device(self.config.device).type == "cuda"
        self._inflight = None        # (requests, their tokens on the device, pinned copy, event) of the step that was launched last
        self._token_ring: list = []
        self._token_next = 0
        self._prev_read = False

    @classmethod
    def from_pretrained(cls, model: Union[str, Path], **kw) -> "Engine":
        return cls(model, **kw)

    def warmup(self, batch_sizes: Optional[Sequence[int]] = None) -> List[int]:
        """With CUDA graphs: capture the decode graphs (of all batch buckets, or of those that hold the given batch sizes)
        before the first request instead of in the middle of serving; the reference captures when its decoder is built
        (src/miniserve/graph_decode.py:45-47). Returns the captured buckets; without graphs, nothing."""
        graphs = self.runner.graphs
        return graphs.warmup(batch_sizes) if graphs is not None else []

    # ------------------------------------------------------------------ the reference's calls
    @property
    def waiting(self):
        return self.scheduler.waiting

    @property
    def running(self):
        return self.scheduler.running

    @property
    def preemptions(self) -> int:
        return self.scheduler.preemptions

    def add_request(self, req: Request) -> Request:
        vocab = self.spec.vocab_size()
        for t in req.prompt_ids:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token {t} is outside the vocabulary of {vocab}")
        SamplingParams(req.temperature, req.top_k, req.top_p).validate()
        self.scheduler.add(req)
        req.arrival_time = self.clock()
        return req

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    def cancel(self, req: Request) -> None:
        """Honoured at the start of the next step (src/miniserve/engine.py:163-177)."""
        req.cancelled = True

    def run_until_idle(self) -> None:
        while self.has_work():
            self.step()
        self._final_check()

    def _final_check(self) -> None:
        """A step without sampled rows (a prompt portion) hands nothing back with which the error word could ride."""
        check = getattr(self.runner.K, "check_device_errors", None)
        if check is not None and self.runner.device.type == "cuda":
            check()

    def step(self) -> StepRecord:
        """One step of the engine. With ``EngineConfig.pipeline`` the tokens a step chooses stay on the device: the next
        step is launched with them (``StepEntry.from_previous``) before the host reads them, so the device never waits for
        the host's book-keeping; what this call emits are then the tokens of the step BEFORE the one it launches. A request
        whose token turns out to be a stop token has by then been given one more row, whose result is dropped."""
        t0 = self.clock()
        prev, self._inflight = self._inflight, None
        try:
            return self._step(prev, t0)
        except BaseException:
            # The step did not happen: the scheduler was not advanced, so the same tokens are planned again next time
            # (pages that were reserved stay with their requests). The tokens of the step before are still unread.
            if prev is not None and self._inflight is None and not self._prev_read:
                self._inflight = prev
            raise

    def _step(self, prev, t0: float) -> StepRecord:
        self._prev_read = False
        plan = self.scheduler.schedule()
        now = self.clock()
        for r in plan.aborted:
            r.finish_reason, r.finish_time = "abort", now
            if self.on_finish:
                self.on_finish(r)
        useful = 0
        if plan.items:
            entries = []
            prev_row = {id(r): i for i, r in enumerate(prev[0])} if prev is not None else {}
            for s in plan.items:
                r = s.req
                if r.admitted_time is None:
                    r.admitted_time = now
                want = (s.count - 1,) if s.samples else ()
                if s.start + s.count > len(r.prompt_ids) + len(r.output_ids):  # its last token is still on the device
                    if s.count != 1 or id(r) not in prev_row:
                        raise RuntimeError(f"request {r.id} was scheduled past its known tokens")
                    entries.append(StepEntry(r.id, [0], s.start, want, from_previous=prev_row[id(r)]))
                else:
                    entries.append(StepEntry(r.id, r.tokens(s.start, s.start + s.count), s.start, want))
            logits = self.runner.step(entries, previous_tokens=prev[1] if prev is not None else None)
            self.scheduler.advance(plan)
            rows = [s.req for s in plan.items if s.samples]
            if rows:
                params = [SamplingParams(r.temperature, r.top_k, r.top_p, self._seed(r)) for r in rows]
                greedy = self.runner.greedy_tokens if len(rows) == len(plan.items) else None
                chosen = self.sampler.sample_device(logits, params, [len(r.output_ids) + r.in_flight for r in rows], greedy)
                flag = self._error_word()
                if self._pipeline:
                    pinned, event = self._token_buffer()
                    pinned[:len(rows)].copy_(chosen, non_blocking=True)
                    if flag is not None:   # the kernels' error word rides with the tokens: reading it costs no wait of its own
                        pinned[-1:].copy_(flag, non_blocking=True)
                    event.record()
                    for r in rows:
                        r.in_flight += 1
                    self._inflight = (rows, chosen, pinned, event)
                else:
                    values = (chosen if flag is None else torch.cat([chosen, flag])).tolist()
                    if flag is not None:
                        self.runner.K.raise_for_error_code(values.pop())
                    for r, tok in zip(rows, values):
                        self._emit(r, int(tok))
                        useful += 1
        if prev is not None:
            self._prev_read = True
            useful += self._read(prev)
        decode = sum(1 for s in plan.items if s.count == 1 and s.start > 0)
        n_tok = plan.num_tokens
        self.prefill_tokens_computed += n_tok - decode
        self.peak_running = max(self.peak_running, len(self.scheduler.running))
        if self.cache.pools:
            self.peak_pages_in_use = max(self.peak_pages_in_use, max(p.capacity - p.num_free for p in self.cache.pools))
        rec = StepRecord(plan.admitted, decode, useful, self.clock() - t0, plan.preempted, n_tok, n_tok - decode)
        self.steps.append(rec)
        return rec

    def _error_word(self):
        """The device word in which a kernel reports that it gave up on a bounded wait (None if these kernels have none)."""
        get = getattr(self.runner.K, "error_flag", None)
        return get(self.runner.device) if get is not None and self.runner.device.type == "cuda" else None

    def _token_buffer(self):
        """A pinned buffer for one step's chosen tokens (and, last, the kernels' error word) and the event of its copy,
        from a ring of three."""
        if not self._token_ring:
            self._token_ring = [(torch.zeros(max(self.config.max_seqs, 1) + 1, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                                for _ in range(3)]
        self._token_next = (self._token_next + 1) % len(self._token_ring)
        return self._token_ring[self._token_next]

    def _read(self, inflight) -> int:
        """Wait for a launched step's tokens and hand them to their requests; returns how many were kept."""
        rows, _, pinned, event = inflight
        event.synchronize()
        code = int(pinned[-1])
        if code:
            pinned[-1] = 0
            self.runner.K.raise_for_error_code(code)  # these tokens, and the cache entries behind them, are not to be trusted
        kept = 0
        for r, tok in zip(rows, pinned[:len(rows)].tolist()):
            r.in_flight -= 1
            if r.state == "finished":
                continue  # ended by the token before this one (a stop token), or cancelled: this row was one too many
            self._emit(r, int(tok))
            kept += 1
        return kept

    def drain(self) -> None:
        """Read the tokens of a step that is still on its way (pipelined engine), launching nothing new."""
        if self._inflight is not None:
            prev, self._inflight = self._inflight, None
            self._read(prev)

    def stats(self) -> dict:
        """src/miniserve/paged_engine.py:68-80."""
        return {
            "prefix_cache": self.cache.prefix_sharing,
            "prefix_tokens_hit": self.cache.shared_tokens,
            "prefill_tokens_computed": self.prefill_tokens_computed,
            "preemptions": self.preemptions,
            "peak_running": self.peak_running,
            "peak_blocks_in_use": self.peak_pages_in_use,
            "pool_blocks": self.cache.pools[0].capacity if self.cache.pools else 0,
            "pool_mib": self.runner.kv_bytes_per_token * self.config.pool_blocks() * self.config.block_size / 2**20,
            "steps": len(self.steps),
        }

    # ------------------------------------------------------------------ internals
    def _seed(self, r: Request) -> int:
        return int(r.seed) if r.seed is not None else (self.config.seed * 1000003 + r.id) & ((1 << 62) - 1)

    def _emit(self, req: Request, tok: int) -> None:
        """src/miniserve/engine.py:279-291: a stop token ends the request and is not kept."""
        now = self.clock()
        if tok in req.eos_ids and not req.ignore_eos:
            self._finish(req, "stop", now)
            return
        req.output_ids.append(tok)
        req.token_times.append(now)
        if req.first_token_time is None:
            req.first_token_time = now
        if self.on_token:
            self.on_token(req, tok)
        if len(req.output_ids) >= req.max_new_tokens:
            self._finish(req, "length", now)

    def _finish(self, req: Request, reason: str, now: float) -> None:
        self.scheduler.finish(req)
        req.finish_reason, req.finish_time = reason, now
        self.finished.append(req)
        if self.on_finish:
            self.on_finish(req)

    # ------------------------------------------------------------------ the Python entry point
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], max_new_tokens: int = 64,
                 eos_ids: Sequence[int] = (), temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 seed: Optional[int] = None) -> Union[GenerationResult, List[GenerationResult]]:
        """Generate for one prompt (a list of token ids) or for several at once (a list of lists).

        Options as src/miniserve/generate.py:85-96. Several prompts run together under the scheduler;
        each result is what the prompt would give alone.
        """
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        batch = [list(prompts)] if single else [list(p) for p in prompts]
        t0 = self.clock()
        reqs = [self.add_request(Request(p, max_new_tokens, tuple(eos_ids), temperature, top_k, top_p,
                                         None if seed is None else seed + i)) for i, p in enumerate(batch)]
        while any(r.state != "finished" for r in reqs):
            self.step()
        self.drain()
        self._final_check()
        total = self.clock() - t0
        out = []
        for r in reqs:
            times = [b - a for a, b in zip(r.token_times, r.token_times[1:])]
            out.append(GenerationResult(r.output_ids, len(r.prompt_ids), (r.first_token_time or self.clock()) - t0, total,
                                        times, r.finish_reason or "length",
                                        self.runner.kv_bytes_per_token * (len(r.prompt_ids) + len(r.output_ids))))
        return out[0] if single else out


def generate(engine: Engine, prompt_ids: Sequence[int], max_new_tokens: int = 64, eos_ids: Sequence[int] = (),
             temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: Optional[int] = None) -> GenerationResult:
    """The reference's ``generate(model, prompt_ids, ...)`` (src/miniserve/generate.py:85) with an engine in the model's place."""
    return engine.generate(list(prompt_ids), max_new_tokens, eos_ids, temperature, top_k, top_p, seed)
