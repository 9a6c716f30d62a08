"""Continuous batching: admission, prompt portions under a token budget, decoding,
finishing, and what happens when pages run out.

Policy (the reference's, src/engine/engine.cpp:53-178, plus portions):

* Admission is first come first served: the head of the waiting queue is admitted while
  fewer than `max_batch` requests run, a state slot is free and the pages of its first
  portion are free; nothing behind a blocked head is looked at.
* A step gives one token to every running request that is decoding, then fills what is
  left of `max_step_tokens` with portions of the prompts (or recomputed contexts) of the
  running requests that are not yet prefilled, oldest first.  All items draw pages from
  one budget; a request whose pages do not fit is left out of this step.
* When no running request can be given anything and more than one is running, the
  youngest request that holds pages is preempted: everything it holds is given back, it
  returns to the front of the waiting queue, and when it is admitted again it recomputes
  prompt + output so far in portions.  Its output continues identically.
* A request that could never fit (prompt + max_tokens beyond one request's share of the
  pool or beyond the position limit) is refused when it is added, instead of spinning
  as the reference does (src/engine/engine.cpp:120-126).
* A step may be planned while the tokens sampled by the step before it are still on their
  way from the GPU (`begin_step` / `resolve_step` instead of `finish_step`): such a request
  counts its pending token in its length, brings a token that the GPU fills in, is left out
  if the pending token is its last, and is never preempted - a plan that would have to
  preempt is given up (`can_preempt=False`), the caller settles the pending tokens and
  plans again.

This file decides only; `Engine` in engine.py runs the plans on the GPU.
"""

from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

from ..cache.manager import CacheManager, RequestCache
from ..sampling.sampler import SamplingParams


class SeqStatus(enum.Enum):
    Waiting = 0
    Running = 1
    Finished = 2


@dataclass
class Sequence_:
    id: int
    prompt: List[int]
    params: SamplingParams
    max_tokens: int
    eos_id: int
    seed: int
    output: List[int] = field(default_factory=list)
    status: SeqStatus = SeqStatus.Waiting
    prefilled: bool = False
    handle: Optional[RequestCache] = None
    preempted: int = 0
    pending: int = 0          # 1 while a sampled token has not been read from the GPU yet
    pending_row: int = -1     # ... and the row of that step's samples it will be found in

    def context(self) -> List[int]:
        return self.prompt + self.output

    def context_length(self) -> int:
        return len(self.prompt) + len(self.output) + self.pending

    def context_slice(self, start: int, stop: int) -> List[int]:
        """context()[start:stop] without building the whole list."""
        n = len(self.prompt)
        if stop <= n:
            return self.prompt[start:stop]
        if start >= n:
            return self.output[start - n:stop - n]
        return self.prompt[start:] + self.output[:stop - n]


PENDING_TOKEN = -1        # placeholder in a plan for a token the GPU still holds


@dataclass
class PlanItem:
    seq: Sequence_
    tokens: List[int]
    samples: bool          # the portion ends the context: logits of its last token are wanted
    was_prefill: bool
    source_row: int = -1   # >= 0: the single token is row source_row of the previous step's samples


def cache_too_small_for_window(cache: CacheManager) -> str:
    """Why a windowed group of the cache could never hold one request's window ('' if each can):
    a query sees its last `window` keys, which may straddle one page more than they fill."""
    for index, group in enumerate(cache.groups):
        window = group.need.window
        if window and group.num_pages < cache.blocks_for(window) + 1:
            return (f"cache group {index} keeps a window of {window} keys and needs "
                    f"{cache.blocks_for(window) + 1} pages for one request, it has {group.num_pages}")
    return ""


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch: int = 256, max_step_tokens: int = 2048,
                 max_positions: int = 0):
        if max_step_tokens <= 0 or max_batch <= 0:
            raise ValueError("max_batch and max_step_tokens must be positive")
        self.cache = cache
        self.max_batch, self.max_step_tokens = max_batch, max_step_tokens
        self.max_positions = max_positions
        self.waiting: Deque[int] = deque()
        self.running: List[int] = []
        self.sequences: Dict[int, Sequence_] = {}
        self.next_id = 0
        self.preemptions = 0

    # ------------------------------------------------------------------ requests
    def add(self, prompt: Sequence[int], params: SamplingParams, max_tokens: int, eos_id: int,
            seed: int) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("Engine: empty prompt")
        if max_tokens <= 0:
            raise ValueError("Engine: max_tokens must be positive")
        total = len(prompt) + max_tokens
        share = self.cache.max_tokens_per_request()
        if total - 1 > share:
            raise ValueError(f"Engine: request needs up to {total - 1} cached tokens, the page "
                             f"pool holds {share} for one request")
        short = cache_too_small_for_window(self.cache)
        if short:
            raise ValueError(f"Engine: {short}")
        if self.max_positions and total - 1 > self.max_positions:
            raise ValueError(f"Engine: request would reach position {total - 1}, the model's "
                             f"limit is {self.max_positions}")
        seq = Sequence_(self.next_id, prompt, params, max_tokens, eos_id, seed)
        self.sequences[seq.id] = seq
        self.waiting.append(seq.id)
        self.next_id += 1
        return seq.id

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _admit(self) -> None:
        cache = self.cache
        while self.waiting and len(self.running) < self.max_batch and cache.can_open():
            seq = self.sequences[self.waiting[0]]
            first = min(seq.context_length(), self.max_step_tokens)
            # pages the first portion needs, seen against what is free before this step; a
            # windowed group gives pages back as the portions pass, so one free page lets the
            # request start and `plan` cuts its portions to the room there is
            if any((1 if group.need.window else cache.blocks_for(first)) > free
                   for group, free in zip(cache.groups, cache.free_pages())):
                break
            self.waiting.popleft()
            seq.handle = cache.open(seq.id)
            seq.status = SeqStatus.Running
            self.running.append(seq.id)

    def plan(self, can_preempt: bool = True) -> List[PlanItem]:
        """Admit, then choose this step's items.  May preempt (unless told not to: then a
        plan that needs a preemption comes back empty).  Returns [] when nothing can run
        (then nothing is running, or a single request waits for nothing: cannot happen for
        requests that passed `add`; or every running request waits for its last token)."""
        self._admit()
        cache = self.cache
        while True:
            items: List[PlanItem] = []
            tokens_left = self.max_step_tokens
            pages_left = cache.free_pages()

            def take(handle, n) -> bool:
                if cache.fits_in_held_pages(handle, n):
                    return True
                need = cache.pages_needed(handle, n)
                if any(k > left for k, left in zip(need, pages_left)):
                    return False
                for g, k in enumerate(need):
                    pages_left[g] -= k
                return True

            for sid in self.running:                      # decodes first
                seq = self.sequences[sid]
                if not seq.prefilled or tokens_left <= 0:
                    continue
                if len(seq.output) + seq.pending >= seq.max_tokens:
                    continue                              # its pending token is its last
                if take(seq.handle, 1):
                    if seq.pending:
                        items.append(PlanItem(seq, [PENDING_TOKEN], True, False, seq.pending_row))
                    else:
                        items.append(PlanItem(seq, [seq.output[-1]], True, False))
                    tokens_left -= 1
            for sid in self.running:                      # then prompt portions
                seq = self.sequences[sid]
                if seq.prefilled or tokens_left <= 0:
                    continue
                total = seq.context_length()
                handle = seq.handle
                if cache.prefix_enabled and handle.length == 0 and not any(handle.tables):
                    # Shared pages are looked for only now that the request gets its first tokens:
                    # the longer it waits, the more of its prefix others have registered.  A
                    # shared page that only the prefix cache held counted as free until this
                    # moment, so what the acquisition pins comes out of this step's budget - and
                    # if earlier items of the step were already promised those pages, the
                    # acquisition is undone and the request waits for the next step.
                    cap = ((total - 1) // cache.page_size) * cache.page_size
                    if cap > 0:
                        before = cache.free_pages()
                        cache.acquire_prefix(handle, seq.context_slice(0, cap))
                        left = [have - (b - a) for have, b, a
                                in zip(pages_left, before, cache.free_pages())]
                        if any(v < 0 for v in left):
                            cache.release_prefix(handle)
                            continue
                        pages_left = left
                remaining = total - handle.length
                chunk = min(remaining, tokens_left)
                # shrink the portion to the pages that are left
                room = min((len(t) + left) * cache.page_size - handle.length
                           for t, left in zip(handle.tables, pages_left)) if handle.tables \
                    else chunk
                chunk = min(chunk, room)
                if chunk <= 0 or not take(handle, chunk):
                    continue
                portion = seq.context_slice(handle.length, handle.length + chunk)
                items.append(PlanItem(seq, portion, chunk == remaining, True))
                tokens_left -= chunk
            if items or len(self.running) <= 1 or not can_preempt or not self._preempt_youngest():
                return items

    def _preempt_youngest(self) -> bool:
        for sid in reversed(self.running):
            seq = self.sequences[sid]
            if not any(page >= 0 for table in seq.handle.tables for page in table):
                continue              # holds no pages; preempting it would free nothing
            self.cache.close(seq.handle)
            seq.handle = None
            seq.prefilled = False
            seq.status = SeqStatus.Waiting
            seq.preempted += 1
            self.running.remove(sid)
            self.waiting.appendleft(sid)
            self.preemptions += 1
            return True
        return False

    # ------------------------------------------------------------------- results
    def finish_step(self, items: Sequence[PlanItem], tokens: Sequence[Optional[int]]) -> None:
        """Record the sampled token of every item that sampled (None for the others), retire
        what is finished and register freshly prefilled pages for sharing."""
        self.begin_step(items)
        self.resolve_step(items, tokens)

    def begin_step(self, items: Sequence[PlanItem]) -> None:
        """The step has been launched: every item that samples now has a token pending, in
        the row of the step's samples that its place among the sampling items gives."""
        row = 0
        for item in items:
            if not item.samples:
                continue
            seq = item.seq
            if seq.status is SeqStatus.Running and seq.handle is not None:
                seq.prefilled = True
                seq.pending, seq.pending_row = 1, row
            row += 1

    def resolve_step(self, items: Sequence[PlanItem], tokens: Sequence[Optional[int]]) -> None:
        """The step's sampled tokens have arrived (None for items that did not sample).  A
        request that an earlier step's token has finished meanwhile is passed over: its item
        ran for nothing."""
        for item, token in zip(items, tokens):
            seq = item.seq
            if not item.samples or seq.status is not SeqStatus.Running or seq.handle is None \
                    or not seq.pending:
                continue
            seq.pending, seq.pending_row = 0, -1
            seq.output.append(int(token))
            hit_eos = seq.eos_id >= 0 and token == seq.eos_id
            if hit_eos or len(seq.output) >= seq.max_tokens:
                seq.status = SeqStatus.Finished
                self.cache.close(seq.handle)
                seq.handle = None
                self.running.remove(seq.id)
            elif item.was_prefill and self.cache.prefix_enabled:
                known = min(seq.handle.length, len(seq.prompt) + len(seq.output))
                self.cache.register_prefix(seq.handle, seq.context_slice(0, known))
