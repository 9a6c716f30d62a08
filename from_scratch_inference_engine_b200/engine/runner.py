"""The step function: one batch of (request, its next tokens) through the model.

`ModelRunner.step` takes portions of prompts and single decoded tokens alike, cut
anywhere.  It runs only the tokens it is given, as one batch, on top of what earlier
steps left in the cache, and returns float32 logits at the places asked for.  It owns
the cache manager and the device memory of the pages and of per-request state.
Counterpart in the reference: Model::forward_batch (src/model/model.cpp:159-281), which
returns the last row of each item only.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..parts.base import LayerCache
from ..parts.model import DecoderModel
from .context import PinnedRing, StepContext
from .runtime import Runtime


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places (indices into these
    tokens) whose logits are wanted."""

    handle: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    # >= 0: the single token is not known on the host yet; it is row `source_row` of the
    # `device_tokens` given to step() (what the step before sampled)
    source_row: int = -1


class DeviceFault(RuntimeError):
    """A kernel met an input it had to refuse (token id or position out of range)."""


DECODE_BATCHES = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)
TABLE_STEP = 64          # block tables of captured steps grow in steps of this many pages


class _DecodeGraph:
    """One decode step (a single token per request) of a fixed batch size and block-table
    width, captured in a CUDA graph.  Its inputs live in one fixed int32 device buffer that
    every step refills with one copy from pinned host memory; requests fewer than the batch
    size are padded with entries that store nothing and see no key."""

    def __init__(self, runner: "ModelRunner", batch: int, width: int):
        self.runner, self.batch, self.width = runner, batch, width
        groups = len(runner.cache.groups)
        ints = 6 * batch + groups * (batch * width + batch)
        device = runner.runtime.device
        self.buffer = torch.zeros(ints, dtype=torch.int32, device=device)
        self.rows = torch.arange(batch, dtype=torch.int32, device=device)
        # scratch of its own: the graph holds raw addresses, so what it uses must never be
        # freed or regrown by later steps
        self.scratch: Dict[str, torch.Tensor] = {}
        self.context = self.fill([], [], [], [[] for _ in range(groups)])
        # one plain run first: libraries initialise, tile lists and scratch get allocated
        stream = torch.cuda.Stream(device=device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            runner.model.forward(self.context, runner.layer_caches, self.rows)
        torch.cuda.current_stream().wait_stream(stream)
        from ..kernels import ops
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launches
        # Nothing may free pinned or device memory while the stream is capturing; the garbage
        # collector would, if it came across a dropped engine's staging buffers just then.
        import gc
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, pool=runner.graph_pool(), capture_error_mode="thread_local"):
                self.logits = runner.model.forward(self.context, runner.layer_caches, self.rows)
        finally:
            if was_enabled:
                gc.enable()
        self.launches = ops.launches - before

    def fill(self, token_ids, pos0, slots, tables) -> StepContext:
        """Write one step's inputs into the fixed buffer (padded to the batch size)."""
        runner, pad = self.runner, self.batch - len(token_ids)
        page = runner.cache.page_size
        group_tables = [(page, list(t) + [[]] * pad) for t in tables]
        return StepContext(runner.runtime, runner._ring, self.scratch, runner.error,
                           list(token_ids) + [0] * pad, list(range(self.batch)),
                           [1] * self.batch, list(pos0) + [0] * pad, list(slots) + [0] * pad,
                           group_tables, table_width=self.width, out=self.buffer,
                           max_context=self.width * page)

    def replay(self) -> torch.Tensor:
        from ..kernels import ops
        self.graph.replay()
        ops.launches += self.launches
        return self.logits


class ModelRunner:
    def __init__(self, model: DecoderModel, runtime: Runtime, page_size: int = 16,
                 num_pages=2048, max_requests: int = 256, enable_prefix_cache: bool = False,
                 cuda_graphs: bool = True, max_step_tokens: int = 8192):
        """`max_step_tokens` and `max_requests` cap what one step may bring (tokens; requests):
        a step beyond them is refused before anything runs, so that the working memory of a
        step is bounded by what `reserve_step_memory` has seen."""
        if max_step_tokens <= 0 or max_requests <= 0:
            raise ValueError("max_step_tokens and max_requests must be positive")
        self.model, self.runtime = model, runtime
        self.max_step_tokens, self.max_step_items = int(max_step_tokens), int(max_requests)
        needs = model.cache_needs()
        self.cache = CacheManager(needs, page_size, num_pages, max_requests, enable_prefix_cache,
                                  has_state=any(n is not None for n in model.state_needs()))
        device, dtype = runtime.device, runtime.dtype
        # pages of group g: [page, entry in group, K or V, kv_head, slot, head_dim]
        self.pages: List[torch.Tensor] = []
        for group in self.cache.groups:
            need = group.need
            self.pages.append(torch.zeros((group.num_pages, len(group.entries), 2, need.kv_heads,
                                           page_size, need.head_dim), dtype=dtype, device=device))
        self.states: List[Optional[torch.Tensor]] = []
        for need in model.state_needs():
            self.states.append(None if need is None else torch.zeros(
                (max_requests, *need.shape), dtype=need.dtype, device=device))
        self.layer_caches: List[LayerCache] = []
        for index, (_, entry, writes) in enumerate(model.schedule):
            cache = LayerCache(writes=writes, state=self.states[index])
            if needs[entry] is not None:
                g, position = self.cache.entry_group[entry]
                pages = self.pages[g]
                cache.group = g
                cache.k_pages = pages[:, position, 0]
                cache.v_pages = pages[:, position, 1]
                cache.page_stride = pages.stride(0)
                cache.pages, cache.entry_index = pages, position
            self.layer_caches.append(cache)
        self.error = runtime.error
        self._ring = PinnedRing()
        self._scratch: Dict[str, torch.Tensor] = {}
        # steps of single tokens replay a captured graph (not for mixers with state of their
        # own, whose Python-side loops a graph would freeze)
        self.cuda_graphs = (cuda_graphs and all(s is None for s in self.states)
                            and getattr(model, "capturable", False))
        self._graphs: Dict[tuple, _DecodeGraph] = {}
        self._graph_pool = None
        self.vocab_size = model.spec.vocab_size
        self.max_positions = runtime.max_positions     # length of the position tables

    # ------------------------------------------------------------------- checks
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise ValueError("step: empty batch")
        if len(entries) > self.max_step_items:
            raise ValueError(f"step: {len(entries)} requests in one step, the runner was built "
                             f"for {self.max_step_items}")
        total = sum(len(entry.tokens) for entry in entries)
        if total > self.max_step_tokens:
            raise ValueError(f"step: {total} tokens in one step, the runner was built for "
                             f"{self.max_step_tokens}")
        seen = set()
        for entry in entries:
            if entry.handle.closed:
                raise ValueError(f"step: request {entry.handle.request_id!r} is closed")
            if id(entry.handle) in seen:
                raise ValueError(f"step: request {entry.handle.request_id!r} appears twice")
            seen.add(id(entry.handle))
            n = len(entry.tokens)
            if n == 0:
                raise ValueError(f"step: request {entry.handle.request_id!r} brings no tokens")
            low, high = (entry.tokens[0], entry.tokens[0]) if n == 1 else \
                (min(entry.tokens), max(entry.tokens))
            if entry.source_row >= 0:
                if n != 1:
                    raise ValueError("step: only a single token can come from the device")
                low = high = 0                    # the embedding kernel checks the id it finds
            if low < 0 or high >= self.vocab_size:
                raise IndexError(f"step: token id out of range [0, {self.vocab_size}) in request "
                                 f"{entry.handle.request_id!r}")
            if entry.handle.length + n > self.max_positions:
                raise ValueError(f"step: request {entry.handle.request_id!r} would reach position "
                                 f"{entry.handle.length + n}, the limit is {self.max_positions}")
            for w in entry.want:
                if not 0 <= w < n:
                    raise IndexError(f"step: wanted place {w} outside the {n} tokens brought")

    def graph_pool(self):
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    def _place_device_tokens(self, ctx: StepContext, entries: Sequence[StepEntry], starts,
                             device_tokens: Optional[torch.Tensor]) -> None:
        """Tokens that the step before sampled go from its result on the device straight into
        this step's ids (entry e's token sits at ids[starts[e]])."""
        pairs = [(starts[e], entry.source_row) for e, entry in enumerate(entries) if entry.source_row >= 0]
        if not pairs:
            return
        if device_tokens is None:
            raise ValueError("step: entries take tokens from the device, but none were given")
        host = np.asarray([d for d, _ in pairs] + [r for _, r in pairs], dtype=np.int32)
        from ..kernels import ops
        ops.place_tokens(ctx.token_ids, self._ring.stage(host, self.runtime.device), device_tokens)

    def reserve_step_memory(self, tokens: int = 0) -> int:
        """Run one step of `tokens` tokens (default: the cap) of a scratch request, so that the
        allocator holds the working memory of the largest step before serving starts and no
        later step has to ask the driver for memory; the request's pages and slot are given
        back.  Skipped (returns 0) when the pool cannot hold that many tokens right now."""
        tokens = min(tokens or self.max_step_tokens, self.max_step_tokens, self.max_positions)
        cache = self.cache
        if not cache.can_open() or any(cache.blocks_for(tokens) > free for free in cache.free_pages()):
            return 0
        handle = cache.open(("reserve_step_memory", id(self)))
        try:
            self.step([StepEntry(handle, [0] * tokens, [tokens - 1])])
            torch.cuda.current_stream().synchronize()
        finally:
            cache.close(handle)
        return tokens

    def capture_decode_graphs(self, max_context: int, max_batch: int = 0) -> int:
        """Capture ahead of time the decode steps that requests of up to `max_context` tokens
        in batches of up to `max_batch` (default: all the runner takes) will replay, instead of
        at their first use in the middle of serving.  Returns how many graphs now exist."""
        if not self.cuda_graphs:
            return 0
        limit = max_batch or self.cache.slots.num_slots
        pages = -(-max(1, max_context) // self.cache.page_size)
        widths = range(TABLE_STEP, -(-pages // TABLE_STEP) * TABLE_STEP + 1, TABLE_STEP)
        for batch in DECODE_BATCHES:
            for width in widths:
                if (batch, width) not in self._graphs:
                    self._graphs[batch, width] = _DecodeGraph(self, batch, width)
            if batch >= limit:
                break
        return len(self._graphs)

    def _decode_step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor]):
        """A step of single tokens through a captured graph: (whether it ran, logits)."""
        cache = self.cache
        count = len(entries)
        batch = next((b for b in DECODE_BATCHES if b >= count), None)
        if batch is None:
            return False, None
        blocks = max((len(t) for e in entries for t in e.handle.tables), default=1)
        width = -(-max(blocks, 1) // TABLE_STEP) * TABLE_STEP
        key = (batch, width)
        graph = self._graphs.get(key)
        if graph is None:
            graph = self._graphs[key] = _DecodeGraph(self, batch, width)
        ctx = graph.fill([max(0, e.tokens[0]) for e in entries], [e.handle.length for e in entries],
                         [e.handle.slot for e in entries],
                         [[e.handle.table_array(g) for e in entries] for g in range(len(cache.groups))])
        self._place_device_tokens(ctx, entries, range(count), device_tokens)
        logits = graph.replay()
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        if not wanted:
            return True, None
        if wanted == list(range(len(wanted))):
            return True, logits[:len(wanted)]
        index = torch.tensor(wanted, dtype=torch.long, device=self.runtime.device)
        return True, logits.index_select(0, index)

    # --------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry],
             device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch; returns float32 logits [wanted places, vocab] in the order of the
        entries and of their `want`, or None when nothing is wanted.  The returned tensor
        may be reused by the next step: read it before stepping again.  `device_tokens`
        (int32, on the device) holds the tokens of entries with a `source_row`."""
        self._validate(entries)
        cache = self.cache
        for entry in entries:
            cache.reserve(entry.handle, len(entry.tokens))
        if self.cuda_graphs and all(len(e.tokens) == 1 for e in entries):
            ran, logits = self._decode_step(entries, device_tokens)
            if ran:
                for entry in entries:
                    cache.commit(entry.handle, 1)
                return logits
        token_ids: List[int] = []
        q_start, q_len, pos0, slots, want_rows = [], [], [], [], []
        fresh_slots = []
        for entry in entries:
            q_start.append(len(token_ids))
            q_len.append(len(entry.tokens))
            pos0.append(entry.handle.length)
            slots.append(entry.handle.slot)
            if entry.handle.fresh_state:          # first step since the slot was acquired
                fresh_slots.append(entry.handle.slot)
                entry.handle.fresh_state = False
            want_rows += [len(token_ids) + w for w in entry.want]
            token_ids += [0] if entry.source_row >= 0 else list(entry.tokens)
        tables = [(cache.page_size, [e.handle.table_array(g) for e in entries])
                  for g in range(len(cache.groups))]
        ctx = StepContext(self.runtime, self._ring, self._scratch, self.error, token_ids, q_start,
                          q_len, pos0, slots, tables)
        self._place_device_tokens(ctx, entries, q_start, device_tokens)
        if fresh_slots and any(s is not None for s in self.states):
            index = torch.tensor(fresh_slots, dtype=torch.long, device=self.runtime.device)
            for state in self.states:
                if state is not None:
                    state.index_fill_(0, index, 0)
        rows = None
        if want_rows:
            rows = self._ring.stage(np.asarray(want_rows, dtype=np.int32), self.runtime.device)
        logits = self.model.forward(ctx, self.layer_caches, rows)
        for entry in entries:
            cache.commit(entry.handle, len(entry.tokens))
        return logits

    def raise_on_device_error(self) -> None:
        code = int(self.error.item())
        if code:
            self.error.zero_()
            self.runtime.reset_after_fault()
            what = {1: "token id outside the vocabulary", 2: "position outside the table",
                    11: "matrix product: the copy engine's stage never became free",
                    12: "matrix product: a tile never arrived", 13: "matrix product: the "
                    "accumulator never completed",
                    21: "tiled matrix product: the copy engine's stage never became free",
                    22: "tiled matrix product: a stage never arrived",
                    23: "tiled matrix product: the accumulator was never read out",
                    24: "tiled matrix product: the accumulator never completed",
                    31: "tcgen05 attention: the copy engine's slot never became free",
                    32: "tcgen05 attention: a tile or the softmax never arrived",
                    33: "tcgen05 attention: scores or outputs never completed",
                    34: "tcgen05 attention: shared memory does not start on a 1,024-byte boundary",
                    35: "tcgen05 decode attention: the copy engine's slot never became free",
                    36: "tcgen05 decode attention: a tile or the softmax never arrived",
                    37: "tcgen05 decode attention: scores or outputs never completed",
                    38: "tcgen05 decode attention: shared memory does not start on a 1,024-byte "
                        "boundary"}
            raise DeviceFault(what.get(code, f"device error flag {code}"))
