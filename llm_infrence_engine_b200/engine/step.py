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

    state: torch.Tensor  # [max_seqs, *shape], float32
    write: bool = True


class StepContext:
    """Everything about the running step that a part may read."""

    def __init__(self, K, dtype, device, page_size: int):
        self.K, self.dtype, self.device, self.page_size = K, dtype, device, page_size
        self.num_tokens = 0
        self.num_seqs = 0
        self.token_ids: torch.Tensor = None      # [N] int32
        self.positions: torch.Tensor = None      # [N] int32, absolute, 0-based
        self.token_seq: torch.Tensor = None      # [N] int32, index of the token's request within the step
        self.seq_slots: torch.Tensor = None      # [R] int32, state slot of each request
        self.block_tables: List[torch.Tensor] = []  # per group [R, max_blocks] int32
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


class ModelRunner:
    def __init__(self, spec: ModelSpec, kernels, cache: CacheManager, group_of_entry: List[Optional[int]],
                 dtype: torch.dtype, device, num_pages: int, page_size: int, max_seqs: int):
        self.spec, self.K, self.cache = spec, kernels, cache
        self.dtype, self.device = dtype, torch.device(device)
        self.page_size, self.max_seqs = page_size, max_seqs
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
                self.bindings.append(StateBinding(torch.zeros((max_seqs,) + tuple(cs.shape), dtype=torch.float32, device=self.device)))
            elif cs is None:
                self.bindings.append(None)
            else:
                raise TypeError(f"cache entry {entry} has a spec of unknown kind {type(cs).__name__}")
        self._staging: List[list] = []  # ring of [pinned buffer, event of the copy that last read it]
        self._next_staging = 0
        self.last_h2d_bytes = 0  # bytes of step inputs copied to the device by the last step

    # ------------------------------------------------------------------ building the step's inputs
    def _build(self, entries: Sequence[StepEntry]) -> tuple:
        cache, ps = self.cache, self.page_size
        groups = len(cache.groups)
        vocab = self.spec.embedding.vocab
        ids: List[int] = []
        pos: List[int] = []
        seq: List[int] = []
        rows: List[int] = []
        starts, lens, ctxs, slots = [], [], [], []
        for r, e in enumerate(entries):
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.req!r} brings no tokens to the step")
            for t in e.tokens:
                if not 0 <= int(t) < vocab:
                    raise ValueError(f"request {e.req!r}: token {t} is outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"request {e.req!r}: wanted place {w} is outside its {n} tokens")
            starts.append(len(ids)); lens.append(n); ctxs.append(e.context_len); slots.append(cache.slot(e.req))
            ids.extend(int(t) for t in e.tokens)
            pos.extend(range(e.context_len, e.context_len + n))
            seq.extend([r] * n)
            rows.extend(starts[-1] + int(w) for w in e.want)
        if len(set(e.req for e in entries)) != len(entries):
            raise ValueError("a request appears twice in one step")
        N, R, M = len(ids), len(entries), len(rows)
        max_blocks = 1
        for e in entries:
            for g in range(groups):
                max_blocks = max(max_blocks, len(cache.block_table(e.req, g)))
        tables: List[List[int]] = []
        mapping: List[List[int]] = []
        for g in range(groups):
            flat_table: List[int] = []
            flat_map: List[int] = []
            for e in entries:
                t = cache.block_table(e.req, g)
                need = -(-(e.context_len + len(e.tokens)) // ps)
                if len(t) < need:
                    raise ValueError(f"request {e.req!r} has {len(t)} pages in group {g} but the step needs {need}")
                flat_table.extend(t)
                flat_table.extend([NULL_PAGE] * (max_blocks - len(t)))
                for p in range(e.context_len, e.context_len + len(e.tokens)):
                    page = t[p // ps]
                    if page == NULL_PAGE:
                        raise ValueError(f"request {e.req!r}: position {p} has no page in group {g}")
                    flat_map.append(page * ps + p % ps)
            tables.append(flat_table)
            mapping.append(flat_map)
        packed = ids + pos + seq + slots + rows
        for g in range(groups):
            packed += mapping[g] + tables[g]
        return packed, N, R, M, max_blocks, starts, lens, ctxs, slots

    def _upload(self, packed: List[int]) -> torch.Tensor:
        """One asynchronous copy of the step's integers from pinned memory. The staging buffers form a
        ring: a buffer is written again only after the copy that last read it has finished, because
        the host may run several steps ahead of the device when nothing is read back in between."""
        n = len(packed)
        self.last_h2d_bytes = 4 * n
        host = torch.tensor(packed, dtype=torch.int32)
        if self.device.type != "cuda":
            return host.to(self.device)
        if not self._staging:
            self._staging = [[None, None] for _ in range(4)]
        slot = self._staging[self._next_staging]
        self._next_staging = (self._next_staging + 1) % len(self._staging)
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0] is None or slot[0].numel() < n:
            slot[0] = torch.empty(max(2 * n, 8192), dtype=torch.int32, pin_memory=True)
        slot[0][:n].copy_(host)
        dev = slot[0][:n].to(self.device, non_blocking=True)
        slot[1] = torch.cuda.Event()
        slot[1].record()
        return dev

    def make_context(self, entries: Sequence[StepEntry]):
        packed, N, R, M, max_blocks, starts, lens, ctxs, slots = self._build(entries)
        dev = self._upload(packed)
        ctx = StepContext(self.K, self.dtype, self.device, self.page_size)
        ctx.num_tokens, ctx.num_seqs = N, R
        o = 0
        ctx.token_ids = dev[o:o + N]; o += N
        ctx.positions = dev[o:o + N]; o += N
        ctx.token_seq = dev[o:o + N]; o += N
        ctx.seq_slots = dev[o:o + R]; o += R
        logit_rows = dev[o:o + M]; o += M
        for g in range(len(self.cache.groups)):
            ctx.slot_mapping.append(dev[o:o + N]); o += N
            ctx.block_tables.append(dev[o:o + R * max_blocks].view(R, max_blocks)); o += R * max_blocks
        ctx.seq_starts, ctx.seq_lens, ctx.seq_context, ctx.seq_slot_list = starts, lens, ctxs, slots
        ctx.max_context = max(c + n for c, n in zip(ctxs, lens))
        ctx.max_seq_len = max(lens)
        return ctx, logit_rows

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries as one batch; returns float32 logits ``[wanted, vocab]`` in the order of the
        entries and of their ``want``, or None if nothing was wanted."""
        if not entries:
            return None
        ctx, logit_rows = self.make_context(entries)
        fresh = [s for s, c in zip(ctx.seq_slot_list, ctx.seq_context) if c == 0]
        if fresh:
            for b in self.bindings:
                if isinstance(b, StateBinding):
                    b.state[fresh] = 0
        return self.forward(ctx, logit_rows)

    def forward(self, ctx: StepContext, logit_rows: torch.Tensor) -> Optional[torch.Tensor]:
        spec = self.spec
        residual = spec.embedding.forward(ctx)
        delta = None
        for call in spec.schedule:
            b = self.bindings[call.cache]
            if b is not None and b.write != call.write:
                b = type(b)(**{**b.__dict__, "write": call.write})
            delta = spec.layers[call.layer].forward(ctx, residual, delta, b)
        if logit_rows.numel() == 0:
            return None
        h = spec.final_norm.norm_rows(ctx, residual, delta, logit_rows)
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
