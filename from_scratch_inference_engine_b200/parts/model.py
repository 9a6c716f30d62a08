"""A decoder model assembled from a `ModelSpec`: embedding, blocks in run order, final
norm and output head."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheNeed
from ..config.spec import ModelSpec
from ..kernels import ops
from ..weights.loader import check_tensors, to_runtime_dtype
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, StateNeed, build_part


class DecoderModel:
    """Embedding -> blocks in the order of `spec.schedule` -> final norm -> head.

    The run order is data: entry i of the schedule runs block `layer` on cache entry
    `cache` (its own by default).  A block named twice runs twice with the same weights;
    a call with writes_cache=False attends over keys another call stored.
    Reference wiring: src/model/model.cpp:159-281.
    """

    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.schedule = spec.resolved_schedule()
        self.blocks = [build_part("arrangement",
                                  _arrangement_spec(layer), layer.prefix) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, spec.final_norm_prefix)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.runtime = None

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> List[TensorSpec]:
        spec = self.spec
        shape = (spec.vocab_size, spec.hidden_size)
        specs = [TensorSpec(spec.embedding_name, shape)]
        if spec.head_name is not None:
            specs.append(TensorSpec(spec.head_name, shape))
        else:
            # a tied head may be stored a second time; it must then equal the embedding
            specs.append(TensorSpec("lm_head.weight", shape, optional=True,
                                    same_as=spec.embedding_name))
        specs += self.final_norm.tensor_specs()
        for block in self.blocks:
            specs += block.tensor_specs()
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        """Check `tensors` (host or device, any stored dtype) against the declarations, move
        them to the runtime's device and dtypes, and hand each part its own."""
        specs = self.tensor_specs()
        check_tensors(specs, tensors)
        by_name = {s.name: s for s in specs}
        placed = {}
        for name, tensor in tensors.items():
            spec = by_name[name]
            if spec.optional and spec.same_as:
                continue
            placed[name] = to_runtime_dtype(tensor, spec, runtime.dtype).to(runtime.device)
        self.runtime = runtime
        self.embedding = placed[self.spec.embedding_name].contiguous()
        self.head = (placed[self.spec.head_name].contiguous()
                     if self.spec.head_name is not None else self.embedding)
        runtime.prepare_weight(self.head)
        self.final_norm.bind(placed, runtime)
        for block in self.blocks:
            block.bind(placed, runtime)

    # -------------------------------------------------------------------- needs
    @property
    def capturable(self) -> bool:
        """Whether a step launches the same kernels whatever the data (every part says so)."""
        return self.final_norm.capturable and all(block.capturable for block in self.blocks)

    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """Need of each cache entry (index = position in the run order); None where the
        entry is not written by its own call or the mixer keeps no keys."""
        needs: List[Optional[CacheNeed]] = [None] * len(self.schedule)
        for index, (layer, entry, writes) in enumerate(self.schedule):
            need = self.blocks[layer].mixer.cache_need()
            if writes:
                needs[entry] = need
            elif need != needs[entry]:
                raise ValueError(f"schedule entry {index} reads cache entry {entry} whose "
                                 f"layout {needs[entry]} differs from its own {need}")
        return needs

    def state_needs(self) -> List[Optional[StateNeed]]:
        """State each call of the run order keeps per request (None for most mixers)."""
        return [self.blocks[layer].mixer.state_need() for layer, _, _ in self.schedule]

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, caches: List[LayerCache], want_rows: Optional[torch.Tensor]):
        """Run the step's tokens; returns float32 logits [len(want_rows), vocab] (None if
        nothing is wanted).  `caches[i]` belongs to call i of the run order."""
        rt = self.runtime
        hidden = self.spec.hidden_size
        x = rt.buffer("model.residual", ctx.num_tokens, hidden, torch.float32)
        ops.embed_gather(ctx.token_ids, self.embedding, x, ctx.error)
        delta = None
        for index, (layer, _, _) in enumerate(self.schedule):
            delta = self.blocks[layer].forward(ctx, x, delta, caches[index])
        if want_rows is None or want_rows.numel() == 0:
            return None
        y = self.final_norm.forward(x, delta, rows=want_rows, write_x=False)
        # the logits live where the last step's lived: whoever gets them reads them (or queues
        # what reads them on this stream) before the next step runs
        return rt.linear_f32_out(y, self.head, "model.logits")


def _arrangement_spec(layer):
    from ..config.spec import PartSpec
    return PartSpec(layer.arrangement, {"layer": layer})


def tensor_specs(spec: ModelSpec) -> List[TensorSpec]:
    """Every tensor a model of this spec reads from a checkpoint (no device needed)."""
    return DecoderModel(spec).tensor_specs()
