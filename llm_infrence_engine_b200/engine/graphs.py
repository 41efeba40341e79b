"""Decode-only steps replayed from CUDA graphs, one graph per padded batch size.

The reference captures its decode forward per batch size {1, 2, 4, ...} with static input buffers
and parks padding rows in a scratch slot (src/miniserve/graph_decode.py:23-86), but only for its
slot cache: its paged path rebuilds block tables on the host every step and cannot be captured
(src/miniserve/engine.py:125-128). Here the block tables already live on the device, one row per
state slot, so the captured step reads them in place; a step's own integers (token, position,
table row, cache slot of every row) are copied into one static buffer before the replay. Padding
rows carry token 0 at position 0, point at a table row of null pages and write their key and value
into the null page, which nobody reads.

A graph fixes the launch shapes, so the number of key slices per token is planned for ``max_len``;
the kernel cuts each token's own keys into that many slices on the device, whatever its length.

Steps that bring prompt portions are launched kernel by kernel from Python, a few hundred launches that take the host
longer than the device needs to run them. Their shape, the tuple of (tokens, wanted rows) per request, often comes
again: a prompt cut under the token budget gives step after step of exactly the budget. So a shape that is seen a
third time is captured too (a handful are kept, the least recently used goes), and from then on such a step is one
launch.
"""
from __future__ import annotations

import gc
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence

import torch

from .step import StepContext, StepEntry, step_layout


def bucket_sizes(max_batch: int) -> List[int]:
    """1, 2, 4, 8, 16, then steps of half a power of two (24, 32, 48, 64, ...) up to and including ``max_batch``.

    The reference pads to powers of two (src/miniserve/graph_decode.py:23-30); above 16 a padded row costs real time
    in the products, so the steps are finer there. A bucket is captured when a batch first needs it.
    """
    out, b = [], 1
    while b < max_batch:
        out.append(b)
        if b >= 16 and b + b // 2 < max_batch:
            out.append(b + b // 2)
        b *= 2
    out.append(max_batch)
    return out


class _Captured:
    def __init__(self, graph, static_in, logits, launches, tokens=None):
        self.graph, self.static_in, self.logits = graph, static_in, logits
        self.launches = launches  # kernels that one replay launches
        self.tokens = tokens      # argmax of every row of ``logits``, made inside the graph (decode graphs)


class DecodeGraphs:
    def __init__(self, runner):
        self.runner = runner
        self.usable = runner.device.type == "cuda" and all(getattr(p, "graph_safe", False) for p in runner.spec.parts())
        self.buckets = bucket_sizes(runner.max_seqs)
        self.captured: Dict[int, _Captured] = {}
        self.shapes: "OrderedDict[tuple, _Captured]" = OrderedDict()  # captured prompt-portion steps, least recently used first
        self.seen: Dict[tuple, int] = {}
        self.max_shapes = 6
        self.capture_after = 3   # a capture costs about a hundred eager steps: only shapes that keep coming are worth it
        self.max_shape_tokens = 8192
        self.pool = None
        self._stream = None
        self.replays = 0
        self.shape_replays = 0

    def fits(self, entries: Sequence[StepEntry]) -> bool:
        return self.usable and len(entries) <= self.buckets[-1] and \
            all(len(e.tokens) == 1 and e.context_len > 0 and len(e.want) == 1 for e in entries)

    def shape_key(self, entries: Sequence[StepEntry]) -> Optional[tuple]:
        """The shape of a step with prompt portions, if such steps may be captured at all."""
        if not self.usable:
            return None
        n = sum(len(e.tokens) for e in entries)
        if n > self.max_shape_tokens or len(entries) > 8:
            return None
        return tuple((len(e.tokens), len(e.want)) for e in entries)

    def run_shape(self, entries: Sequence[StepEntry], previous_tokens: Optional[torch.Tensor] = None):
        """Replays (capturing first, if this is the second time) the graph of this step's shape; returns ``(handled, logits)``."""
        key = self.shape_key(entries)
        if key is None:
            return False, None
        r = self.runner
        cap = self.shapes.get(key)
        if cap is None:
            self.seen[key] = self.seen.get(key, 0) + 1
            if self.seen[key] < self.capture_after:
                if len(self.seen) > 256:
                    self.seen.clear()
                return False, None
        packed, N, R, M, changed, starts, lens, ctxs, slots = r._build(entries)
        static_len = step_layout(N, R, M, len(r.cache.groups))["end"][0]
        if cap is None:
            static_in = torch.zeros(static_len, dtype=torch.int32, device=r.device)
            full = r._upload(packed)
            static_in.copy_(full[:static_len])
            r._sync_tables(full, changed)
            ctx = StepContext(r.K, r.dtype, r.device, r.page_size)
            rows = r._fill_context(ctx, static_in, N, R, M)
            ctx.seq_starts, ctx.seq_lens, ctx.seq_context, ctx.seq_slot_list = starts, lens, ctxs, slots
            ctx.max_context, ctx.max_seq_len = r.max_len, max(lens)
            r.feed(ctx, entries, previous_tokens)
            cap = self._capture_context(ctx, rows)
            cap.static_in = static_in
            self.shapes[key] = cap
            while len(self.shapes) > self.max_shapes:
                self.shapes.popitem(last=False)
        else:
            self.shapes.move_to_end(key)
            full = r._upload(packed)
            cap.static_in.copy_(full[:static_len])
            r._sync_tables(full, changed)
            if any(e.from_previous is not None for e in entries):
                lay = step_layout(N, R, M, len(r.cache.groups))
                if previous_tokens is None:
                    raise ValueError("an entry takes its token from the previous step, but no previous tokens were given")
                r.K.feed_tokens(cap.static_in[:N], cap.static_in[lay["feed"][0]:lay["feed"][0] + N], previous_tokens)
        cap.graph.replay()
        self.shape_replays += 1
        return True, cap.logits

    def _capture_context(self, ctx: StepContext, rows: torch.Tensor) -> _Captured:
        """Warm up, then capture ``forward`` on a context whose tensors are views of a static buffer."""
        r = self.runner
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ctx._tables.clear()
            r.forward(ctx, rows)  # once outside the capture: whatever this shape allocates or sets up for the first time
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        ctx._tables.clear()
        before = r.K.launches
        graph, logits = self._record(lambda: r.forward(ctx, rows))
        return _Captured(graph, None, logits, r.K.launches - before)

    def _record(self, fn):
        """Runs ``fn`` under stream capture; returns ``(graph, what fn returned)``.

        Nothing but the step's own kernels may touch CUDA while the stream is capturing. Python's cyclic collector could: an
        old runner's graphs, found to be garbage in the middle of the capture, are destroyed with a CUDA call that the capture
        forbids and that invalidates it. So the collector is off until the capture ends. (The capture is begun and ended by
        hand: the library's context manager runs a full collection and empties the allocator's cache first, which costs tens
        of milliseconds in a process with a large heap, many times the capture itself.)"""
        graph = torch.cuda.CUDAGraph()
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        if self._stream is None:
            self._stream = torch.cuda.Stream()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            torch.cuda.synchronize()
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                graph.capture_begin(pool=self.pool, capture_error_mode="relaxed")
                try:
                    out = fn()
                finally:
                    graph.capture_end()
            torch.cuda.current_stream().wait_stream(self._stream)
        finally:
            if was_enabled:
                gc.enable()
        return graph, out

    def _layout_len(self, B: int) -> int:
        return step_layout(B, B, B, len(self.runner.cache.groups))["end"][0]

    def _capture(self, B: int) -> _Captured:
        r = self.runner
        static_in = torch.zeros(self._layout_len(B), dtype=torch.int32, device=r.device)
        ctx = StepContext(r.K, r.dtype, r.device, r.page_size)
        rows = r._fill_context(ctx, static_in, B, B, B)
        ctx.seq_starts, ctx.seq_lens, ctx.seq_context = list(range(B)), [1] * B, [1] * B
        ctx.seq_slot_list = [r.max_seqs] * B
        ctx.max_context, ctx.max_seq_len = r.max_len, 1
        # padding values, so that warm-up and capture run on harmless inputs
        lay = step_layout(B, B, B, len(r.cache.groups))
        static_in[lay["tok_slot"][0]:lay["tok_slot"][0] + B] = r.max_seqs
        static_in[lay["slots"][0]:lay["slots"][0] + B] = r.max_seqs   # padding requests own the spare row of every per-request array
        static_in[lay["starts"][0]:lay["starts"][0] + B + 1] = torch.arange(B + 1, dtype=torch.int32, device=r.device)
        static_in[lay["rows"][0]:lay["rows"][0] + B] = torch.arange(B, dtype=torch.int32, device=r.device)
        static_in[lay["feed"][0]:lay["feed"][0] + B] = -1
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                ctx._tables.clear()
                r.K.argmax(r.forward(ctx, rows))
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        ctx._tables.clear()
        before = r.K.launches

        def step():
            logits = r.forward(ctx, rows)
            return logits, r.K.argmax(logits)  # greedy rows need nothing more than this; the others are sampled from ``logits``

        graph, (logits, tokens) = self._record(step)
        return _Captured(graph, static_in, logits, r.K.launches - before, tokens)


    @torch.inference_mode()
    def warmup(self, batch_sizes: Optional[Sequence[int]] = None) -> List[int]:
        """Captures the decode graphs of these batch sizes (all buckets if none are named) now rather than when a batch
        first needs them, as the reference does when its decoder is built (src/miniserve/graph_decode.py:45-47).
        Returns the buckets that are captured afterwards."""
        if not self.usable:
            return []
        wanted = self.buckets if batch_sizes is None else sorted({next(b for b in self.buckets if b >= n)
                                                                  for n in batch_sizes if 0 < n <= self.buckets[-1]})
        for B in wanted:
            if B not in self.captured:
                self.captured[B] = self._capture(B)
        return sorted(self.captured)

    @torch.inference_mode()
    def run(self, entries: Sequence[StepEntry], previous_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        r = self.runner
        n = len(entries)
        B = next(b for b in self.buckets if b >= n)
        if B not in self.captured:
            self.captured[B] = self._capture(B)
        cap = self.captured[B]
        packed, N, R, M, changed, *_ = r._build(entries, pad_to=B)
        dev = r._upload(packed, into=cap.static_in) if not changed else None
        if changed:
            # rows of block tables ride behind the step's own integers: stage everything once, then split on the device
            full = r._upload(packed)
            cap.static_in.copy_(full[: self._layout_len(B)])
            r._sync_tables(full, changed)
        if any(e.from_previous is not None for e in entries):
            if previous_tokens is None:
                raise ValueError("an entry takes its token from the previous step, but no previous tokens were given")
            lay = step_layout(B, B, B, len(r.cache.groups))
            r.K.feed_tokens(cap.static_in[:B], cap.static_in[lay["feed"][0]:lay["feed"][0] + B], previous_tokens)
        cap.graph.replay()
        self.replays += 1
        r.greedy_tokens = cap.tokens[:n]
        return cap.logits[:n]
