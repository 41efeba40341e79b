"""The step function: one flat batch of (request, its next tokens) through the model, from the cache.

A step holds any mix of prompt portions (cut anywhere) and single decoded tokens. It runs only the
tokens it is given, reads everything earlier from the cache, writes the new keys and values into
the requests' pages, and returns the logits at the places that were asked for. The reference's
forward takes a rectangle ``[B, T]`` plus a cache view with five methods and is called once per
prefill and once per decode batch (src/miniserve/model.py:208-237, src/miniserve/paged.py:184-217);
none of that is carried over.

``ModelRunner`` owns the device side of the cache (the page pools of every group, the fixed-size
state tensors) and the model's parts; the host side (which request holds which page and slot) is
the ``CacheManager`` it is given. Whoever drives it (scheduler, replay) admits, reserves and frees
there, and hands ``step`` a list of ``StepEntry``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.spec import NULL_PAGE, FixedStateSpec, PagedKVSpec
from ..models.spec import ModelSpec


@dataclass
class StepEntry:
    req: Hashable                 # the request, as the cache manager knows it
    tokens: Sequence[int]         # its next tokens
    context_len: int              # tokens of it that are already in the cache
    want: Sequence[int] = ()      # places among ``tokens`` whose logits are asked for
    from_previous: Optional[int] = None  # the entry's single token is row ``from_previous`` of the device tensor of tokens
                                         # given to ``step(previous_tokens=...)``; ``tokens`` then holds a placeholder


@dataclass
class PagedKVBinding:
    """What a paged mixer gets for one call: this cache entry's pools and the group its tables belong to."""

    group: int
    k: torch.Tensor  # [num_pages, num_kv_heads, page_size, head_dim]
    v: torch.Tensor
    write: bool = True


@dataclass
class StateBinding:
    """What a mixer with fixed-size state gets: ``state[slot]`` is the request's own, zero at its first token."""

    state: torch.Tensor  # [max_seqs + 1, *shape], float32 (the last row belongs to the padding rows of a captured step)
    write: bool = True


class StepContext:
    """Everything about the running step that a part may read."""

    def __init__(self, K, dtype, device, page_size: int):
        self.K, self.dtype, self.device, self.page_size = K, dtype, device, page_size
        self.num_tokens = 0
        self.num_seqs = 0
        self.token_ids: torch.Tensor = None      # [N] int32
        self.positions: torch.Tensor = None      # [N] int32, absolute, 0-based
        self.token_seq: torch.Tensor = None      # [N] int32, the token's row in the block tables (= its request's state slot)
        self.seq_slots: torch.Tensor = None      # [R] int32, state slot of each request
        self.seq_starts_dev: torch.Tensor = None  # [R + 1] int32, first row of each request in the flat batch, then N
        self.feed_rows: torch.Tensor = None       # [N] int32, row of the previous step's tokens a token comes from, or -1
        self.block_tables: List[torch.Tensor] = []  # per group [state slots + 1, max_blocks] int32, a row per state slot
        self.slot_mapping: List[torch.Tensor] = []  # per group [N] int32: page * page_size + offset of the token's key
        self.seq_starts: List[int] = []          # host: first row of each request in the flat batch
        self.seq_lens: List[int] = []            # host: rows of each request
        self.seq_context: List[int] = []         # host: tokens of each request already cached
        self.seq_slot_list: List[int] = []       # host copy of seq_slots
        self.max_context = 0                     # host: longest context_len + rows over the requests
        self.max_seq_len = 0                     # host: most rows of one request
        self._tables: Dict[tuple, object] = {}

    def position_tables(self, encoding):
        key = encoding.key()
        if key not in self._tables:
            self._tables[key] = encoding.tables(self)
        return self._tables[key]


def step_layout(N: int, R: int, M: int, groups: int) -> Dict[str, tuple]:
    """Where each array of a step lies in the packed int32 buffer: name -> (offset, length). Block-table rows that
    changed ride behind ``end``."""
    out, o = {}, 0
    for name, n in (("ids", N), ("pos", N), ("tok_slot", N), ("slots", R), ("starts", R + 1), ("rows", M), ("feed", N)):
        out[name] = (o, n)
        o += n
    for g in range(groups):
        out[f"map{g}"] = (o, N)
        o += N
    out["end"] = (o, 0)
    return out


class ModelRunner:
    def __init__(self, spec: ModelSpec, kernels, cache: CacheManager, group_of_entry: List[Optional[int]],
                 dtype: torch.dtype, device, num_pages: int, page_size: int, max_seqs: int, max_len: int,
                 cuda_graphs: bool = False):
        self.spec, self.K, self.cache = spec, kernels, cache
        self.dtype, self.device = dtype, torch.device(device)
        self.page_size, self.max_seqs, self.max_len = page_size, max_seqs, max_len
        self.bindings: List[object] = []
        self.kv_bytes_per_token = 0
        specs = spec.cache_specs()
        for entry, cs in enumerate(specs):
            if isinstance(cs, PagedKVSpec):
                shape = (num_pages, cs.num_kv_heads, page_size, cs.head_dim)
                k = torch.zeros(shape, dtype=dtype, device=self.device)
                v = torch.zeros(shape, dtype=dtype, device=self.device)
                self.bindings.append(PagedKVBinding(group_of_entry[entry], k, v))
                self.kv_bytes_per_token += 2 * cs.num_kv_heads * cs.head_dim * k.element_size()
            elif isinstance(cs, FixedStateSpec):
                self.bindings.append(StateBinding(torch.zeros((max_seqs + 1,) + tuple(cs.shape), dtype=torch.float32, device=self.device)))
            elif cs is None:
                self.bindings.append(None)
            else:
                raise TypeError(f"cache entry {entry} has a spec of unknown kind {type(cs).__name__}")
        # Block tables live on the device, one row per state slot (plus a last row of null pages that padding
        # rows of a captured graph point at); a row is sent again only when the request's table has changed.
        self.max_blocks = max(1, -(-max_len // page_size))
        groups = len(cache.groups)
        self.tables_dev = [torch.zeros((max_seqs + 1, self.max_blocks), dtype=torch.int32, device=self.device) for _ in range(groups)]
        self._synced = [[-1] * max_seqs for _ in range(groups)]
        self._staging: List[list] = []  # ring of [pinned buffer, event of the copy that last read it]
        self._next_staging = 0
        self.last_h2d_bytes = 0  # bytes of step inputs copied to the device by the last step
        if hasattr(kernels, "reserve_transient") and self.device.type == "cuda" and dtype == torch.bfloat16:
            widest = max((p.shape[0] for part in spec.parts() for p in part.params().values() if p.kind == "matrix"
                          and part is not spec.embedding and part is not spec.head), default=0)
            if widest:
                kernels.reserve_transient(widest, self.device)
        self.greedy_tokens = None
        self.graphs = None
        if cuda_graphs:
            from .graphs import DecodeGraphs

            self.graphs = DecodeGraphs(self)

    # ------------------------------------------------------------------ building the step's inputs
    def _build(self, entries: Sequence[StepEntry], pad_to: int = 0):
        """The step's integers as one int32 array plus its layout. ``pad_to`` > 0 (decode-only steps replayed
        from a graph) pads the batch to that many rows with tokens that write to the null page."""
        cache, ps = self.cache, self.page_size
        groups = len(cache.groups)
        vocab = self.spec.embedding.vocab
        R = len(entries)
        if len(set(e.req for e in entries)) != R:
            raise ValueError("a request appears twice in one step")
        lens = [len(e.tokens) for e in entries]
        ctxs = [int(e.context_len) for e in entries]
        slots = [cache.slot(e.req) for e in entries]
        for e, n in zip(entries, lens):
            if n == 0:
                raise ValueError(f"request {e.req!r} brings no tokens to the step")
            if e.context_len + n > self.max_len:
                raise ValueError(f"request {e.req!r} would reach {e.context_len + n} tokens, more than max_len {self.max_len}")
        if max(lens) == 1:
            return self._build_single_tokens(entries, ctxs, slots, pad_to)
        ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if ids.min() < 0 or ids.max() >= vocab:
            bad = int(ids[(ids < 0) | (ids >= vocab)][0])
            raise ValueError(f"token {bad} is outside the vocabulary of {vocab}")
        pos = np.concatenate([np.arange(c, c + n, dtype=np.int64) for c, n in zip(ctxs, lens)])
        starts = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int64)
        tok_slot = np.repeat(np.asarray(slots, dtype=np.int64), lens)
        rows: List[int] = []
        for st, e, n in zip(starts, entries, lens):
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"request {e.req!r}: wanted place {w} is outside its {n} tokens")
                rows.append(int(st) + int(w))
        N, M = int(ids.shape[0]), len(rows)
        pad = max(0, pad_to - N)
        feed = np.full(N + pad, -1, np.int64)
        for st, e, n in zip(starts, entries, lens):
            if e.from_previous is not None:
                if n != 1:
                    raise ValueError(f"request {e.req!r}: only a single token can come from the previous step's tokens")
                feed[int(st)] = int(e.from_previous)
        parts = [ids, np.zeros(pad, np.int64), pos, np.zeros(pad, np.int64), tok_slot, np.full(pad, self.max_seqs, np.int64),
                 np.asarray(slots, dtype=np.int64), np.full(pad, self.max_seqs, np.int64),
                 starts, np.arange(N, N + pad + 1, dtype=np.int64),
                 np.asarray(rows, dtype=np.int64), np.arange(N, N + pad, dtype=np.int64) if pad_to else np.zeros(0, np.int64),
                 feed]
        changed = []  # (group, slot, offset of the row in the packed array)
        offset = sum(len(p) for p in parts)
        for g in range(groups):
            maps = []
            for e, c, n in zip(entries, ctxs, lens):
                t = cache.block_table(e.req, g)
                if len(t) * ps < c + n:
                    raise ValueError(f"request {e.req!r} has {len(t)} pages in group {g} but the step needs {-(-(c + n) // ps)}")
                if n == 1:
                    pages = np.asarray([t[c // ps]], dtype=np.int64)
                    p = np.asarray([c], dtype=np.int64)
                else:
                    p = np.arange(c, c + n, dtype=np.int64)
                    first = c // ps
                    pages = np.asarray(t[first:(c + n - 1) // ps + 1], dtype=np.int64)[p // ps - first]
                if (pages == NULL_PAGE).any():
                    raise ValueError(f"request {e.req!r}: a position of the step has no page in group {g}")
                maps.append(pages * ps + p % ps)
            parts += maps + [np.zeros(pad, np.int64)]
            offset += N + pad
        for g in range(groups):
            for e, slot in zip(entries, slots):
                v = cache.table_version(e.req, g)
                if self._synced[g][slot] != v:
                    t = cache.block_table(e.req, g)
                    if len(t) > self.max_blocks:
                        raise ValueError(f"request {e.req!r} holds {len(t)} pages, more than max_len allows")
                    row = np.zeros(self.max_blocks, np.int64)
                    row[:len(t)] = t
                    parts.append(row)
                    changed.append((g, slot, offset, v))
                    offset += self.max_blocks
        packed = np.concatenate(parts).astype(np.int32)
        return packed, N + pad, R + pad, M + (pad if pad_to else 0), changed, [int(x) for x in starts], lens, ctxs, slots

    def _build_single_tokens(self, entries, ctxs, slots, pad_to: int):
        """``_build`` for steps in which every request brings one token (decoding): plain lists, one array at the end."""
        cache, ps = self.cache, self.page_size
        groups = len(cache.groups)
        vocab = self.spec.embedding.vocab
        R = len(entries)
        ids = [int(e.tokens[0]) for e in entries]
        for t in ids:
            if not 0 <= t < vocab:
                raise ValueError(f"token {t} is outside the vocabulary of {vocab}")
        rows = []
        for i, e in enumerate(entries):
            for w in e.want:
                if int(w) != 0:
                    raise ValueError(f"request {e.req!r}: wanted place {w} is outside its 1 tokens")
                rows.append(i)
        pad = max(0, pad_to - R)
        zeros = [0] * pad
        feed = [-1 if e.from_previous is None else int(e.from_previous) for e in entries] + [-1] * pad
        packed = (ids + zeros + ctxs + zeros + slots + [self.max_seqs] * pad + slots + [self.max_seqs] * pad + list(range(R + pad + 1)) + rows
                  + (list(range(R, R + pad)) if pad_to else []) + feed)
        for g in range(groups):
            for e, c in zip(entries, ctxs):
                t = cache.block_table(e.req, g)
                page = t[c // ps] if c // ps < len(t) else NULL_PAGE
                if page == NULL_PAGE:
                    raise ValueError(f"request {e.req!r}: position {c} has no page in group {g}")
                packed.append(page * ps + c % ps)
            packed += zeros
        changed = []
        tables = []
        offset = len(packed)
        for g in range(groups):
            for e, slot in zip(entries, slots):
                v = cache.table_version(e.req, g)
                if self._synced[g][slot] != v:
                    t = cache.block_table(e.req, g)
                    if len(t) > self.max_blocks:
                        raise ValueError(f"request {e.req!r} holds {len(t)} pages, more than max_len allows")
                    row = np.zeros(self.max_blocks, np.int32)
                    row[:len(t)] = t
                    tables.append(row)
                    changed.append((g, slot, offset, v))
                    offset += self.max_blocks
        arr = np.asarray(packed, dtype=np.int32)
        if tables:
            arr = np.concatenate([arr] + tables)
        M = len(rows) + (pad if pad_to else 0)
        return arr, R + pad, R + pad, M, changed, list(range(R)), [1] * R, ctxs, slots

    def _stage(self, packed: "np.ndarray") -> torch.Tensor:
        """The pinned buffer that holds ``packed`` for one asynchronous copy. The buffers form a ring: one is
        written again only after the copy that last read it has finished, because the host may run
        several steps ahead of the device when nothing is read back in between."""
        n = int(packed.shape[0])
        self.last_h2d_bytes = 4 * n
        if not self._staging:
            self._staging = [[None, None, None] for _ in range(4)]  # pinned tensor, event of its last copy, numpy view
        slot = self._staging[self._next_staging]
        self._next_staging = (self._next_staging + 1) % len(self._staging)
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0] is None or slot[0].numel() < n:
            slot[0] = torch.empty(max(2 * n, 8192), dtype=torch.int32, pin_memory=True)
            slot[2] = slot[0].numpy()
            slot[1] = torch.cuda.Event()
        slot[2][:n] = packed
        self._last_slot = slot
        return slot[0][:n]

    def _upload(self, packed: "np.ndarray", into: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.device.type != "cuda":
            dev = torch.from_numpy(packed).to(self.device)
            if into is not None:
                into[: dev.numel()].copy_(dev)
                return into
            return dev
        pinned = self._stage(packed)
        if into is not None:
            into[: pinned.numel()].copy_(pinned, non_blocking=True)
            dev = into
        else:
            dev = pinned.to(self.device, non_blocking=True)
        self._last_slot[1].record()
        return dev

    def _sync_tables(self, dev: torch.Tensor, changed) -> None:
        for g, slot, off, version in changed:
            self.tables_dev[g][slot].copy_(dev[off:off + self.max_blocks])
            self._synced[g][slot] = version

    def make_context(self, entries: Sequence[StepEntry], pad_to: int = 0, into: Optional[torch.Tensor] = None):
        packed, N, R, M, changed, starts, lens, ctxs, slots = self._build(entries, pad_to)
        dev = self._upload(packed, into)
        self._sync_tables(dev, changed)
        ctx = StepContext(self.K, self.dtype, self.device, self.page_size)
        logit_rows = self._fill_context(ctx, dev, N, R, M)
        ctx.seq_starts, ctx.seq_lens, ctx.seq_context, ctx.seq_slot_list = starts, lens, ctxs, slots
        ctx.max_context = max(c + n for c, n in zip(ctxs, lens))
        ctx.max_seq_len = max(lens)
        return ctx, logit_rows

    def _fill_context(self, ctx: StepContext, dev: torch.Tensor, N: int, R: int, M: int) -> torch.Tensor:
        """Point the context's tensors at their places in the packed device array (``step_layout``)."""
        ctx.num_tokens, ctx.num_seqs = N, R
        lay = step_layout(N, R, M, len(self.cache.groups))

        def view(name):
            o, n = lay[name]
            return dev[o:o + n]

        ctx.token_ids, ctx.positions, ctx.token_seq = view("ids"), view("pos"), view("tok_slot")
        ctx.seq_slots, ctx.seq_starts_dev = view("slots"), view("starts")
        ctx.feed_rows = view("feed")
        ctx.slot_mapping, ctx.block_tables = [], []
        for g in range(len(self.cache.groups)):
            ctx.slot_mapping.append(view(f"map{g}"))
            ctx.block_tables.append(self.tables_dev[g])
        return view("rows")

    def feed(self, ctx: StepContext, entries: Sequence[StepEntry], previous_tokens: Optional[torch.Tensor]) -> None:
        """Fill in the tokens that come from the step before (``StepEntry.from_previous``), on the device."""
        if any(e.from_previous is not None for e in entries):
            if previous_tokens is None:
                raise ValueError("an entry takes its token from the previous step, but no previous tokens were given")
            self.K.feed_tokens(ctx.token_ids, ctx.feed_rows, previous_tokens)

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], previous_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run the entries as one batch; returns float32 logits ``[wanted, vocab]`` in the order of the
        entries and of their ``want``, or None if nothing was wanted. ``previous_tokens``: int32 tokens on the device
        that entries with ``from_previous`` take their token from (the step before chose them; the host need not have
        read them yet)."""
        if not entries:
            return None
        self.greedy_tokens = None  # set by a captured decode step: the argmax of the returned rows, already on the device
        if self.graphs is not None:
            if self.graphs.fits(entries):
                return self.graphs.run(entries, previous_tokens)
            handled, logits = self.graphs.run_shape(entries, previous_tokens)
            if handled:
                return logits
        ctx, logit_rows = self.make_context(entries)
        self.feed(ctx, entries, previous_tokens)
        return self.forward(ctx, logit_rows)

    def forward(self, ctx: StepContext, logit_rows: torch.Tensor) -> Optional[torch.Tensor]:
        """The model on the step's batch. If anything raises in the middle, the kernels object is told to drop what the
        unfinished step left with it (``abandon_step``), so that the next step, of whatever request or runner, starts clean."""
        try:
            return self._forward(ctx, logit_rows)
        except BaseException:
            abandon = getattr(self.K, "abandon_step", None)
            if abandon is not None:
                abandon()
            raise

    def _forward(self, ctx: StepContext, logit_rows: torch.Tensor) -> Optional[torch.Tensor]:
        spec = self.spec
        for b in self.bindings:   # a request's fixed-size state starts from zero: decided on the device, so captured steps do it too
            if isinstance(b, StateBinding):
                self.K.zero_fresh_state(b.state, ctx.seq_slots, ctx.seq_starts_dev, ctx.positions)
        residual = spec.embedding.forward(ctx)
        for call in spec.schedule:
            b = self.bindings[call.cache]
            if b is not None and b.write != call.write:
                b = type(b)(**{**b.__dict__, "write": call.write})
            spec.layers[call.layer].forward(ctx, residual, b)
        if logit_rows.numel() == 0:
            if hasattr(self.K, "flush"):
                self.K.flush()  # nothing reads the residual stream any more: an addition that was put off must not stay behind
            return None
        h = spec.final_norm.norm_rows(ctx, residual, logit_rows)
        return spec.head.forward(ctx, h)

    # ------------------------------------------------------------------ accounting
    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a decode step reads: every tensor once; the embedding table only through the
        output head that shares it (a step gathers a few of its rows)."""
        spec = self.spec
        n = 0
        for part in spec.parts():
            if part is spec.embedding:
                continue
            n += part.weight_bytes()
        if spec.head.tied_to is not None:
            n += spec.embedding.weight_bytes()
        return n


def group_layout(specs: Sequence[object]):
    """Distinct ``PagedKVSpec`` values in order of appearance, and for every cache entry its group (None if not paged)."""
    groups: List[PagedKVSpec] = []
    of_entry: List[Optional[int]] = []
    for cs in specs:
        if isinstance(cs, PagedKVSpec):
            if cs not in groups:
                groups.append(cs)
            of_entry.append(groups.index(cs))
        else:
            of_entry.append(None)
    return groups, of_entry
