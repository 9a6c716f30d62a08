"""The step context: the batch of one step as device arrays every part can read.

It is mixer-agnostic: tokens packed end to end, their absolute positions, one record
per request (where its tokens start, how many, its first position, its state slot), and
per cache group the block tables and the physical slot of every new token.  All of it
reaches the device in one copy from pinned host memory.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class GroupStep:
    page_size: int
    block_tables: torch.Tensor      # int32 [items, max_blocks], -1 where no page is held
    slot_of: torch.Tensor           # int32 [tokens], page * page_size + offset of each new token


@dataclass
class Tiles:
    item: torch.Tensor              # int32 [count]
    row0: torch.Tensor              # int32 [count]
    count: int


class PinnedRing:
    """Pinned staging buffers used in turn; a buffer is reused only after the copy that last
    read it has finished.  Deep enough that the copies of two steps never meet: a step is
    staged while the step before it still runs, and waiting for a buffer would stall the host
    until the GPU has caught up."""

    def __init__(self, depth: int = 32):
        self.depth = depth
        self.buffers: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.next = 0
        self.bytes_staged = 0        # host-to-device bytes so far (benchmarks read this)

    def stage(self, host: np.ndarray, device: torch.device,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Copy `host` (int32) to the device; into the front of `out` when given (a fixed
        buffer that a captured graph reads), else into fresh device memory."""
        i = self.next
        self.next = (i + 1) % self.depth
        if self.events[i] is not None:
            self.events[i].synchronize()
        n = host.size
        if self.buffers[i] is None or self.buffers[i].numel() < n:
            self.buffers[i] = torch.empty(max(n, 1024) * 2, dtype=torch.int32).pin_memory()
        staging = self.buffers[i][:n]
        staging.numpy()[:] = host
        self.bytes_staged += n * 4
        if out is None:
            out = staging.to(device, non_blocking=True)
        else:
            out = out[:n]
            out.copy_(staging, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[i] = event
        return out


class StepContext:
    def __init__(self, runtime, ring: PinnedRing, scratch: Dict[str, torch.Tensor],
                 error: torch.Tensor, token_ids: Sequence[int], q_start: Sequence[int],
                 q_len: Sequence[int], pos0: Sequence[int], slots: Sequence[int],
                 group_tables: Sequence[Tuple[int, List[List[int]]]],
                 table_width: int = 0, out: Optional[torch.Tensor] = None,
                 max_context: int = 0):
        """group_tables: per cache group (page_size, block table of each item).
        table_width forces the width of the device block tables, `out` is a fixed device
        buffer to fill instead of fresh memory, max_context overrides the longest context
        (all three serve captured graphs, whose shapes and launch choices must not vary)."""
        self.runtime = runtime
        self._ring, self._scratch, self.error = ring, scratch, error
        self.num_tokens = T = len(token_ids)
        self.num_items = I = len(q_len)
        self.h_qstart = np.asarray(q_start, dtype=np.int32)
        self.h_qlen = np.asarray(q_len, dtype=np.int32)
        self.h_pos0 = np.asarray(pos0, dtype=np.int32)
        self.h_slots = np.asarray(slots, dtype=np.int32)
        self.max_context = max_context or (int((self.h_pos0 + self.h_qlen).max()) if I else 0)
        self.fixed_context = max_context
        if T == I:                   # one token per request: a decode step
            positions, token_item = self.h_pos0, np.arange(I, dtype=np.int32)
        else:
            positions = np.concatenate([np.arange(p, p + n, dtype=np.int32)
                                        for p, n in zip(pos0, q_len)]) if I else np.zeros(0, np.int32)
            token_item = np.repeat(np.arange(I, dtype=np.int32), self.h_qlen)
        parts = [np.asarray(token_ids, dtype=np.int32), positions, self.h_qstart, self.h_qlen,
                 self.h_pos0, self.h_slots]
        shapes = []
        for page_size, tables in group_tables:
            width = table_width or max(1, max((len(t) for t in tables), default=1))
            table = np.full((I, width), -1, dtype=np.int32)
            for i, row in enumerate(tables):          # rows are lists or ready int32 arrays
                table[i, :len(row)] = row
            block = positions // page_size
            page = table[token_item, block] if T else np.zeros(0, np.int32)
            slot_of = np.where(page >= 0, page * page_size + positions % page_size, -1)
            parts += [table.reshape(-1), slot_of.astype(np.int32)]
            shapes.append((page_size, width))
        flat = np.concatenate(parts) if parts else np.zeros(0, np.int32)
        dev = ring.stage(flat, runtime.device, out)
        self.staged_ints = flat.size
        cut = 0

        def take(n):
            nonlocal cut
            view = dev[cut:cut + n]
            cut += n
            return view
        self.token_ids, self.positions = take(T), take(T)
        self.item_qstart, self.item_qlen = take(I), take(I)
        self.item_pos0, self.item_slots = take(I), take(I)
        self.groups: List[GroupStep] = []
        for page_size, width in shapes:
            tables = take(I * width).view(I, width)
            self.groups.append(GroupStep(page_size, tables, take(T)))
        self._tiles: Dict[Tuple[int, int], Tiles] = {}

    def attention_tiles(self, group_size: int, rows_per_tile: int) -> Tiles:
        """Tiles of `rows_per_tile` query rows, a row being (token, head of the group):
        row = token_in_item * group_size + head_in_group.  No tile spans two items."""
        key = (group_size, rows_per_tile)
        if key not in self._tiles:
            counts = (self.h_qlen.astype(np.int64) * group_size + rows_per_tile - 1) // rows_per_tile
            item = np.repeat(np.arange(self.num_items, dtype=np.int32), counts)
            first = np.cumsum(counts) - counts
            row0 = (np.arange(int(counts.sum())) - np.repeat(first, counts)) * rows_per_tile
            dev = self._ring.stage(np.concatenate([item, row0.astype(np.int32)]),
                                   self.runtime.device)
            n = item.size
            self._tiles[key] = Tiles(dev[:n], dev[n:2 * n], n)
        return self._tiles[key]

    def attention_row_classes(self, group_size: int, class_rows):
        """Requests sorted into row classes by their number of query rows (new tokens x
        group size): class c takes those that fit one tile of class_rows[c] rows, the last
        class takes the rest in as many tiles as needed.  Returns, per non-empty class,
        (class index, Tiles, int32 device list of the class's tokens, their count, the
        longest context in the class)."""
        key = ("classes", group_size, tuple(class_rows))
        if key in self._tiles:
            return self._tiles[key]
        rows = self.h_qlen.astype(np.int64) * group_size
        last = len(class_rows) - 1
        which = np.full(self.num_items, last, dtype=np.int64)
        for c in range(last - 1, -1, -1):
            which[rows <= class_rows[c]] = c
        host, layout = [], []
        for c, per_tile in enumerate(class_rows):
            members = np.nonzero(which == c)[0]
            if members.size == 0:
                continue
            counts = (rows[members] + per_tile - 1) // per_tile
            item = np.repeat(members.astype(np.int32), counts)
            first = np.cumsum(counts) - counts
            row0 = ((np.arange(int(counts.sum())) - np.repeat(first, counts)) * per_tile)
            if item.size > 1:
                # tiles that see the most keys first: blocks start in list order, and the longest
                # should not start last
                last_row = np.minimum(row0 + per_tile, rows[item]) - 1
                keys = self.h_pos0[item] + last_row // group_size + 1
                order = np.argsort(-keys, kind="stable")
                item, row0 = item[order], row0[order]
            tokens = np.concatenate([np.arange(self.h_qstart[i], self.h_qstart[i] + self.h_qlen[i],
                                               dtype=np.int32) for i in members])
            longest = self.fixed_context or int((self.h_pos0[members] + self.h_qlen[members]).max())
            layout.append((c, item.size, tokens.size, longest))
            host += [item, row0.astype(np.int32), tokens]
        dev = self._ring.stage(np.concatenate(host), self.runtime.device)
        out, cut = [], 0
        for c, n_tiles, n_tokens, longest in layout:
            tiles = Tiles(dev[cut:cut + n_tiles], dev[cut + n_tiles:cut + 2 * n_tiles], n_tiles)
            cut += 2 * n_tiles
            out.append((c, tiles, dev[cut:cut + n_tokens], n_tokens, longest))
            cut += n_tokens
        self._tiles[key] = out
        return out

    def scratch(self, name: str, numel: int) -> torch.Tensor:
        """Float32 scratch memory that lives across steps (grown when a step needs more)."""
        have = self._scratch.get(name)
        if have is None or have.numel() < numel:
            have = torch.empty(max(numel, 1), dtype=torch.float32, device=self.runtime.device)
            self._scratch[name] = have
        return have
