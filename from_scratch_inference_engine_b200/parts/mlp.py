"""Dense SwiGLU feed-forward."""

from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Part, register_part


@register_part("feed_forward", "swiglu")
class SwiGluMlp(Part):
    """down( silu(gate(y)) * up(y) ), no biases (reference: src/model/model.cpp:136-140,
    src/model/nn.cpp:74-88).  gate and up are one product over the stacked weight
    [2 * intermediate, hidden]: gate rows first, then up rows."""

    capturable = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int):
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [TensorSpec(p + "gate_proj.weight", (i, h)),
                TensorSpec(p + "up_proj.weight", (i, h)),
                TensorSpec(p + "down_proj.weight", (h, i))]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate_proj.weight"],
                                    tensors[p + "up_proj.weight"]]).contiguous()
        self.w_down = tensors[p + "down_proj.weight"].contiguous()
        runtime.prepare_weight(self.w_gate_up, swiglu=True)
        runtime.prepare_weight(self.w_down)

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        rt = self.runtime
        # the activation and the result are dead when the next feed-forward of the model runs
        return rt.linear(rt.linear_swiglu(y, self.w_gate_up, "swiglu.act"), self.w_down, None, "swiglu.down")
