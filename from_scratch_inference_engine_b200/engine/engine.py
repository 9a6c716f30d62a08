"""The engine a user drives: requests in, tokens out, one GPU step at a time.

Same control surface as the reference's `Engine` (include/engine/engine.hpp:39-89,
bindings/module.cpp:104-147): add_request, step, has_work, output, status, preemptions,
prefix_hits, generate - with the same option names and defaults (block_size, num_blocks,
seed, max_batch, enable_prefix_cache; max_tokens = 16, eos_id = -1 disables the stop).

Steps overlap (`pipeline=True`, the default): `step()` plans and launches the next batch
while the tokens that the batch before it sampled are still on their way to the host -
their ids enter the new batch on the device - and only then waits for them and records
them.  The GPU therefore does not idle while Python plans, stages and launches, and
`output()` lags one step behind the GPU.  The tokens are the same as without the overlap:
a request whose pending token turns out to be its end of sequence has run one token for
nothing, which is dropped.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import List, Optional, Sequence

import torch

from ..config.registry import load_config
from ..parts.model import DecoderModel
from ..sampling.sampler import Sampler, SamplingParams, request_seed
from ..weights.loader import load_checkpoint
from .runner import ModelRunner, StepEntry
from .runtime import Runtime, parse_dtype
from .scheduler import Scheduler, SeqStatus


class LoadedModel:
    """A model bound to its weights on one GPU (the reference's `Model.from_pretrained`,
    bindings/module.cpp:66-79)."""

    def __init__(self, config, model: DecoderModel, runtime: Runtime):
        self.config, self.model, self.runtime = config, model, runtime

    @classmethod
    def from_pretrained(cls, model_dir, dtype="bfloat16", device="cuda:0",
                        max_positions: int = 0, **runtime_options) -> "LoadedModel":
        """Read config.json (which names the architecture) and model.safetensors."""
        config = load_config(model_dir)
        return cls.from_tensors(config, load_checkpoint(model_dir), dtype, device, max_positions,
                                **runtime_options)

    @classmethod
    def from_tensors(cls, config, tensors, dtype="bfloat16", device="cuda:0",
                     max_positions: int = 0, **runtime_options) -> "LoadedModel":
        spec = config.build_spec()
        # positions the engine can encode: what the configuration names (the reference parses
        # max_position_embeddings and never enforces it, src/model/model_config.cpp:25) and
        # at least what the caller's cache will hold
        limit = max(spec.max_position, max_positions) or 32768
        runtime = Runtime(device, parse_dtype(dtype), max_positions=limit, **runtime_options)
        model = DecoderModel(spec)
        model.bind(tensors, runtime)
        return cls(config, model, runtime)

    @classmethod
    def from_random(cls, config, seed: int = 0, std: float = 0.02, dtype="bfloat16",
                    device="cuda:0", max_positions: int = 0, **runtime_options) -> "LoadedModel":
        """Random weights drawn on the device (no folder is written): N(0, std) matrices and
        biases, gains 1 + N(0, std), rounded to bfloat16 first so that both compute dtypes see
        the same numbers.  For benchmarks at sizes whose checkpoint would take minutes to
        write and read back."""
        from ..parts.model import tensor_specs
        from ..weights.random_init import random_tensors_on_device
        tensors = random_tensors_on_device(tensor_specs(config.build_spec()), seed, std, device)
        return cls.from_tensors(config, tensors, dtype, device, max_positions, **runtime_options)

    def forward(self, ids: Sequence[int]) -> torch.Tensor:
        """Logits [len(ids), vocab] of one whole sequence (bindings/module.cpp:70-76)."""
        pages = -(-len(ids) // 16) + 1
        if len(ids) > self.runtime.max_positions:
            raise ValueError(f"forward: {len(ids)} tokens exceed the position table "
                             f"({self.runtime.max_positions})")
        runner = ModelRunner(self.model, self.runtime, page_size=16, num_pages=pages,
                             max_requests=1, max_step_tokens=max(1, len(ids)))
        handle = runner.cache.open(0)
        logits = runner.step([StepEntry(handle, list(ids), list(range(len(ids))))])
        runner.raise_on_device_error()
        return logits.clone()          # a step's logits live in working memory that the next step reuses


class Engine:
    def __init__(self, model: LoadedModel, block_size: int = 16, num_blocks: int = 2048,
                 seed: int = 0, max_batch: int = 256, enable_prefix_cache: bool = False,
                 max_step_tokens: int = 2048, pipeline: bool = True):
        self.model = model
        self.runner = ModelRunner(model.model, model.runtime, page_size=block_size,
                                  num_pages=num_blocks, max_requests=max_batch,
                                  enable_prefix_cache=enable_prefix_cache,
                                  max_step_tokens=max_step_tokens)
        self.scheduler = Scheduler(self.runner.cache, max_batch, max_step_tokens,
                                   self.runner.max_positions)
        self.sampler = Sampler(model.runtime.device)
        self.seed = int(seed)
        self.pipeline = bool(pipeline)
        self._in_flight = None          # (items, Picked) of a launched step whose tokens are not read yet
        self.steps = 0
        self.tokens_prefilled = 0
        self.tokens_decoded = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    max_tokens: int = 16, eos_id: int = -1) -> int:
        params = params or SamplingParams()
        vocab = self.runner.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise IndexError(f"Engine: token id out of range [0, {vocab})")
        rid = self.scheduler.next_id
        seed = params.seed if params.seed is not None else request_seed(self.seed, rid)
        return self.scheduler.add(prompt, params, max_tokens, eos_id, seed)

    def warm_up(self, max_context: int = 0) -> int:
        """Before serving starts: run one step of the largest size (its working memory then
        stays with the allocator) and capture the decode graphs for contexts of up to
        `max_context` tokens (default: what one request may hold); returns their number."""
        if not self.has_work():
            self.runner.reserve_step_memory()
        limit = max_context or min(self.runner.cache.max_tokens_per_request(), self.runner.max_positions)
        return self.runner.capture_decode_graphs(limit, self.scheduler.max_batch)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._in_flight is not None

    def output(self, request_id: int) -> List[int]:
        return self.scheduler.sequences[request_id].output

    def status(self, request_id: int) -> SeqStatus:
        return self.scheduler.sequences[request_id].status

    def preemptions(self) -> int:
        return self.scheduler.preemptions

    def prefix_hits(self) -> int:
        return self.runner.cache.prefix_hits

    # ---------------------------------------------------------------------- step
    def step(self) -> int:
        """One batched step; returns the number of tokens it ran (0 = nothing could run)."""
        if not self.pipeline:
            items = self.scheduler.plan()
            if not items:
                return 0
            picked = self._launch(items)
            tokens = self._tokens_of(items, picked)
            self.scheduler.finish_step(items, tokens)
            return self._count(items)
        # plan and launch the next step before the one in flight is read; a plan that would
        # have to preempt (or finds nothing to do) waits until the pending tokens are settled
        settled = 0
        items = self.scheduler.plan(can_preempt=self._in_flight is None)
        if not items and self._in_flight is not None:
            settled = self._settle()
            items = self.scheduler.plan()
        if not items:
            return settled
        picked = self._launch(items)
        if self._in_flight is not None:
            self._settle()
        self.scheduler.begin_step(items)
        if picked is None:                     # nothing sampled: nothing to wait for
            self.scheduler.resolve_step(items, [None] * len(items))
        else:
            self._in_flight = (items, picked)
        return self._count(items)

    def _launch(self, items):
        """Queue the step on the GPU; returns the sampled tokens' handle (None: no item samples)."""
        entries = [StepEntry(item.seq.handle, item.tokens,
                             [len(item.tokens) - 1] if item.samples else [], item.source_row)
                   for item in items]
        before = self._in_flight[1].device if self._in_flight is not None else None
        logits = self.runner.step(entries, before)
        sampling = [item for item in items if item.samples]
        if not sampling:
            return None
        return self.sampler.sample_async(logits, [i.seq.params for i in sampling],
                                         [i.seq.seed for i in sampling],
                                         [len(i.seq.output) + i.seq.pending for i in sampling],
                                         self.runner.error)

    def _tokens_of(self, items, picked) -> List[Optional[int]]:
        if picked is None:
            return [None] * len(items)
        chosen = iter(picked.result())
        if picked.fault:            # a kernel refused an input or gave up a wait: the ids mean nothing
            self.runner.raise_on_device_error()
        return [next(chosen) if item.samples else None for item in items]

    def _settle(self) -> int:
        """Wait for the tokens of the step in flight and record them."""
        items, picked = self._in_flight
        self._in_flight = None
        self.scheduler.resolve_step(items, self._tokens_of(items, picked))
        return sum(len(item.tokens) for item in items)

    def _count(self, items) -> int:
        self.steps += 1
        for item in items:
            if item.was_prefill:
                self.tokens_prefilled += len(item.tokens)
            else:
                self.tokens_decoded += 1
        return sum(len(item.tokens) for item in items)

    def generate(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                 max_tokens: int = 16, eos_id: int = -1) -> List[int]:
        """Drive the engine until one fresh request completes; returns its tokens."""
        rid = self.add_request(prompt, params, max_tokens, eos_id)
        while self.status(rid) is not SeqStatus.Finished:
            if self.step() == 0:
                raise RuntimeError("Engine: no request can make progress")
        return list(self.output(rid))

    def run_until_done(self) -> None:
        while self.has_work():
            if self.step() == 0:
                raise RuntimeError("Engine: no request can make progress")

    def stats(self) -> dict:
        return {"steps": self.steps, "tokens_prefilled": self.tokens_prefilled,
                "tokens_decoded": self.tokens_decoded, "preemptions": self.preemptions(),
                "prefix_hits": self.prefix_hits(),
                "free_pages": self.runner.cache.free_pages()}
