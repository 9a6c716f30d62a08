"""Arrangements: how a layer's parts are wired around the residual stream."""

from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import LayerSpec
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Part, build_part, register_part
from .norm import RMSNorm


@register_part("arrangement", "prenorm")
class PreNormBlock(Part):
    """x += mixer(norm(x)); x += feed_forward(norm(x))  (src/model/model.cpp:107-141).

    The residual stream `x` is float32 and is updated in place.  A sublayer's output is
    not added at once: it is handed on as `delta` and added by the next norm kernel, which
    reads and writes x anyway.  forward returns the feed-forward's output as the new delta.
    """

    def __init__(self, prefix: str, layer: LayerSpec):
        self.prefix = prefix
        self.mixer_norm = build_part("norm", layer.mixer_norm, prefix + layer.mixer_norm_name)
        self.mixer = build_part("mixer", layer.mixer, prefix + layer.mixer_name)
        self.feed_forward_norm = build_part("norm", layer.feed_forward_norm,
                                            prefix + layer.feed_forward_norm_name)
        self.feed_forward = build_part("feed_forward", layer.feed_forward,
                                       prefix + layer.feed_forward_name)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    @property
    def capturable(self) -> bool:
        return all(part.capturable for part in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(tensors, runtime)

    def forward(self, ctx, x: torch.Tensor, delta: Optional[torch.Tensor],
                cache: LayerCache) -> torch.Tensor:
        # the normed rows are read by the sublayer that follows and by nothing after it
        y = self._normed(self.mixer_norm, x, delta, "prenorm.mixer_in")
        mixed = self.mixer.forward(ctx, y, cache)
        y = self._normed(self.feed_forward_norm, x, mixed, "prenorm.feed_forward_in")
        return self.feed_forward.forward(ctx, y)

    @staticmethod
    def _normed(norm, x, delta, tag):
        """A norm of this package is told where its result may live; any other norm part has the
        plain interface forward(x, delta)."""
        if isinstance(norm, RMSNorm):
            return norm.forward(x, delta, tag=tag)
        return norm.forward(x, delta)
