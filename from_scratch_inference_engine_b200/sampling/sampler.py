"""Greedy and temperature / top-k / top-p sampling on the device.

Options as the reference's `SamplingParams` (include/engine/sampler.hpp:9-13):
temperature (<= 0 selects the first largest logit), top_k (0 = off), top_p (>= 1 =
off), applied in that order (src/sampler/sampler.cpp:25-88).  Unlike the reference,
whose requests share one generator so that a request's tokens depend on what else is
in the batch (src/engine/engine.cpp:131-135), every draw here is a function of
(request seed, index of the output token): a request gives the same tokens alone, in
any batch, and when it is recomputed after a preemption.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops

_MASK = 0xFFFFFFFFFFFFFFFF


@dataclass
class SamplingParams:
    temperature: float = 1.0     # <= 0 selects greedy (argmax)
    top_k: int = 0               # 0 disables top-k
    top_p: float = 1.0           # >= 1 disables top-p (nucleus)
    seed: Optional[int] = None   # None: derived from the engine seed and the request id

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


def _splitmix(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_draw(seed: int, index: int) -> float:
    """The uniform number in [0, 1) of output token `index` of a request with `seed`."""
    bits = _splitmix(_splitmix(seed & _MASK) ^ ((index + 1) * 0xD6E8FEB86659FD93 & _MASK))
    return float(np.float32((bits >> 40) / float(1 << 24)))   # 24 bits: exact in float32, < 1


def request_seed(engine_seed: int, request_id: int) -> int:
    return _splitmix((engine_seed & _MASK) ^ _splitmix(request_id + 0x51ED270B))


class Picked:
    """The tokens one sampling call chose: on the device at once (`device`, int32 [rows]), on
    the host after `result()`, which waits for the copy that was started with the call."""

    def __init__(self, device: torch.Tensor, host: np.ndarray, event, rows: int,
                 watches_fault: bool = False):
        self.device, self._host, self._event, self.rows = device, host, event, rows
        self._watches_fault = watches_fault
        self._list: Optional[List[int]] = None
        self.fault = 0          # after result(): the device's error flag as it stood after the kernels

    def result(self) -> List[int]:
        if self._list is None:
            self._event.synchronize()
            self._list = self._host[:self.rows].tolist()
            if self._watches_fault:
                self.fault = int(self._host[-1])
        return self._list


class Sampler:
    """Chooses one token per row of logits with the device kernels."""

    HOST_BUFFERS = 4           # pinned result buffers in rotation: a result is read at most two calls later

    def __init__(self, device):
        self.device = torch.device(device)
        self._scratch = None
        self._pinned: List[torch.Tensor] = []
        self._turn = 0
        from ..engine.context import PinnedRing
        self._ring = PinnedRing()    # staging of the sampling parameters
        self.bytes_to_device = 0     # sampling parameters copied in (benchmarks read these)
        self.bytes_to_host = 0       # chosen ids copied out

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               seeds: Sequence[int], indices: Sequence[int]) -> List[int]:
        """logits float32 [rows, vocab]; row r is output token indices[r] of a request whose
        seed is seeds[r].  Returns the chosen ids (one device-to-host copy of rows ints)."""
        return self.sample_async(logits, params, seeds, indices).result()

    def _host_buffer(self, rows: int) -> torch.Tensor:
        if not self._pinned or self._pinned[0].numel() - 1 < rows:
            size = max(256, 1 << (rows - 1).bit_length())
            # one more element: the device's error flag travels with the ids
            self._pinned = [torch.zeros(size + 1, dtype=torch.int32, pin_memory=True)
                            for _ in range(self.HOST_BUFFERS)]
        self._turn = (self._turn + 1) % self.HOST_BUFFERS
        return self._pinned[self._turn]

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     seeds: Sequence[int], indices: Sequence[int],
                     error: Optional[torch.Tensor] = None) -> Picked:
        """The same without waiting: the kernels and the copy to pinned host memory are queued,
        the chosen ids stay on the device for a step that feeds them back in.  `error` (int32
        [1], the flag that kernels set when they refuse an input or give up a wait) is copied
        along, so that whoever reads the ids learns of a fault without a transfer of its own."""
        rows = logits.shape[0]
        if rows != len(params):
            raise ValueError("one SamplingParams per row of logits is needed")
        picks = torch.empty((2, rows), dtype=torch.int32, device=self.device)
        any_greedy = any(p.greedy for p in params)
        any_random = any(not p.greedy for p in params)
        if any_greedy:
            need = 2 * rows * ops.ARGMAX_PARTS
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(max(need, 4096), dtype=torch.float32,
                                            device=self.device)
            ops.argmax(logits, picks[0], self._scratch)
        if any_random:
            # one staged copy from pinned memory for all parameters: a copy from pageable memory
            # would wait for the stream and with it for the step that is still running
            host = np.empty((5, rows), dtype=np.float32)
            top_k = host[3].view(np.int32)
            for r, p in enumerate(params):
                host[0, r] = p.temperature if not p.greedy else 0.0
                host[1, r] = min(p.top_p, 1.0)
                host[2, r] = uniform_draw(seeds[r], indices[r])
                top_k[r] = max(0, int(p.top_k))
                host[4, r] = 1.0 if p.greedy else 0.0
            staged = self._ring.stage(host.reshape(-1).view(np.int32), self.device).view(5, rows)
            dev = staged.view(torch.float32)
            self.bytes_to_device += host.nbytes
            ops.sample(logits, dev[0], staged[3], dev[1], dev[2], picks[1])
            chosen = torch.where(dev[4] > 0, picks[0], picks[1]) if any_greedy else picks[1]
        else:
            chosen = picks[0]
        pinned = self._host_buffer(rows)
        pinned[:rows].copy_(chosen, non_blocking=True)
        if error is not None:
            pinned[-1:].copy_(error, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.bytes_to_host += 4 * rows + (4 if error is not None else 0)
        return Picked(chosen, pinned.numpy(), event, rows, error is not None)
