"""Architecture-neutral description of a decoder model.

A model is data: which parts each layer is made of (`LayerSpec`), in which order
the layers run and whose cache they use (`LayerCall`), and which tensors hold the
embedding and the output head.  An architecture's configuration class turns its
own config.json keys into a `ModelSpec`; nothing below this level knows the
architecture's name.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part (mixer, feed-forward, norm, position encoding) by kind and parameters.

    `kind` is looked up in the registry of its role; `params` are passed to the
    part's constructor as keyword arguments, so every size and constant a part
    uses arrives here and none is fixed in the part's code.
    """

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def with_params(self, **extra: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(extra)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerSpec:
    """The parts of one layer and the prefix of its tensor names."""

    prefix: str                      # e.g. "model.layers.3."
    arrangement: str                 # kind of block, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    # tensor-name prefixes of the four parts below `prefix`
    mixer_name: str = "mixer."
    feed_forward_name: str = "feed_forward."
    mixer_norm_name: str = "mixer_norm."
    feed_forward_norm_name: str = "feed_forward_norm."


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    `layer` indexes `ModelSpec.layers` (the weights that run).  `cache` names the
    cache entry the mixer reads; by default a call owns the entry with its own
    position in the schedule.  `writes_cache=False` makes the mixer read that
    entry without appending to it (it must then be written by an earlier call).
    """

    layer: int
    cache: Optional[int] = None
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int                      # 0 = no limit given by the configuration
    embedding_name: str                    # tensor [vocab, hidden]
    head_name: Optional[str]               # tensor [vocab, hidden]; None = reuse the embedding
    final_norm: PartSpec
    final_norm_prefix: str
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[LayerCall, ...]

    def resolved_schedule(self) -> List[Tuple[int, int, bool]]:
        """(layer, cache entry, writes) per call with defaults filled in and checked."""
        out: List[Tuple[int, int, bool]] = []
        written = set()
        for index, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule entry {index} names layer {call.layer}, "
                                 f"the model has {len(self.layers)}")
            entry = index if call.cache is None else call.cache
            if not 0 <= entry < len(self.schedule):
                raise ValueError(f"schedule entry {index} names cache entry {entry} "
                                 f"outside the schedule")
            if call.writes_cache:
                if entry in written:
                    raise ValueError(f"cache entry {entry} is written twice "
                                     f"(schedule entry {index})")
                written.add(entry)
            elif entry not in written:
                raise ValueError(f"schedule entry {index} reads cache entry {entry} "
                                 f"before any call has written it")
            out.append((call.layer, entry, call.writes_cache))
        return out
