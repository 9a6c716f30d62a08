"""Interfaces of the parts a layer is put together from, and their registries.

Roles: "norm", "position", "mixer", "feed_forward", "arrangement".  A part is built
from a `PartSpec` (kind + keyword parameters) and a tensor-name prefix; it declares
the tensors it needs, takes them at `bind`, and runs on a `StepContext`.  No part
knows which model it is in: sizes and constants come from the parameters, the batch
and the cache come from the context.

    class Norm:           forward(x, delta, rows=None, write_x=True) -> y
    class PositionEncoding: prepare(runtime, capacity); fields rotary_dim, table
    class Mixer:          cache_need() -> CacheNeed | None
                          state_need() -> StateNeed | None
                          forward(ctx, y, cache: LayerCache) -> [tokens, hidden]
    class FeedForward:    forward(ctx, y) -> [tokens, hidden]
    class Arrangement:    forward(ctx, x, delta, cache) -> delta'
                          (x is the float32 residual stream, updated in place; delta is
                          the output of the previous sublayer not yet added to x)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..cache.manager import CacheNeed
from ..config.spec import PartSpec
from ..weights.tensor_spec import TensorSpec

ROLES = ("norm", "position", "mixer", "feed_forward", "arrangement")
_REGISTRY: Dict[str, Dict[str, type]] = {role: {} for role in ROLES}


def register_part(role: str, kind: str) -> Callable[[type], type]:
    """Class decorator: make `kind` buildable in `role`."""
    if role not in _REGISTRY:
        raise ValueError(f"unknown role '{role}' (roles: {', '.join(ROLES)})")

    def decorate(cls: type) -> type:
        _REGISTRY[role][kind] = cls
        return cls
    return decorate


def unregister_part(role: str, kind: str) -> None:
    _REGISTRY[role].pop(kind, None)


def registered_parts(role: str) -> List[str]:
    return sorted(_REGISTRY[role])


def build_part(role: str, spec: PartSpec, prefix: str):
    try:
        cls = _REGISTRY[role][spec.kind]
    except KeyError:
        raise KeyError(f"no {role} of kind '{spec.kind}' is registered "
                       f"(registered: {', '.join(registered_parts(role))})") from None
    return cls(prefix=prefix, **spec.params)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size that a mixer keeps: one tensor of `shape` per
    request, zero when the request starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What one call of the run order sees of the cache.

    group        index of the cache group (ctx.groups[group] has the block tables)
    k_pages      view starting at page 0 of this entry's keys; page p begins
                 p * page_stride elements further; layout [kv_head][slot][head_dim]
    v_pages      the same for values
    writes       whether this call stores the new tokens' keys and values
    state        [num_slots, *StateNeed.shape] or None
    pages        the group's page tensor [pages, entries, K|V, kv_heads, slots, head_dim] that
                 k_pages and v_pages are views of (TMA-fed kernels address it as a whole)
    entry_index  which of a page's entries this cache entry is
    """

    group: int = -1
    k_pages: Optional[torch.Tensor] = None
    v_pages: Optional[torch.Tensor] = None
    page_stride: int = 0
    writes: bool = True
    state: Optional[torch.Tensor] = None
    pages: Optional[torch.Tensor] = None     # the group's whole page tensor
    entry_index: int = 0                     # index of this entry inside a page of the group


class Part:
    """Base of all parts: tensor declarations and binding."""

    prefix: str = ""
    # True when forward launches the same kernels on the same addresses whatever the data
    # holds (no host read of a device value, no loop over its values).  Only a model all of
    # whose parts say so has its decode steps captured in CUDA graphs; a part says nothing
    # and is safe.
    capturable: bool = False

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        """Take this part's tensors (already on the device, in their runtime dtypes)."""
        self.runtime = runtime


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None
