"""RMSNorm fused with the residual add that precedes it."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Part, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * gain over the last axis, a plain gain (not 1 + gain),
    statistics in 32-bit (reference: src/model/nn.cpp:45-72, 64-bit statistics there).

    forward adds `delta` into the float32 residual `x` first (one kernel, one pass over x).
    """

    capturable = True

    def __init__(self, prefix: str, width: int, eps: float):
        self.prefix, self.width, self.eps = prefix, int(width), float(eps)
        self.gain: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.prefix + "weight", (self.width,), role="vector", init="gain")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        self.gain = tensors[self.prefix + "weight"].contiguous()

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None, write_x: bool = True,
                tag: Optional[str] = None) -> torch.Tensor:
        """`tag`: where the result may live (`Runtime.buffer`); None asks for fresh memory."""
        count = x.shape[0] if rows is None else rows.numel()
        out = self.runtime.buffer(tag, count, self.width, self.runtime.dtype)
        return ops.add_rmsnorm(x, delta, self.gain, self.eps, out, rows=rows, write_x=write_x)
