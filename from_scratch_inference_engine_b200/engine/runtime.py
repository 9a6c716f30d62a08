"""What the parts get from the engine: device, compute dtype, matrix products, shared tables."""

from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F

from ..kernels import ops

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {name}")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype '{name}' (bfloat16 or float32)") from None


class Runtime:
    """Device and precision of one engine.

    bfloat16: matrix products by the library (cuBLAS through torch, bf16 operands, 32-bit
    accumulation), as the reference engine uses the library for its products
    (src/cuda/device.cu:322-357).  float32: every product by the engine's own FFMA kernel,
    no tensor-core mode.  Everything that is not a plain matrix product is a kernel of
    this package in both modes.
    """

    def __init__(self, device="cuda:0", dtype=torch.bfloat16, max_positions: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this engine has no CPU path")
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        self.max_positions = int(max_positions)
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._tables: Dict[object, torch.Tensor] = {}
        self._f32_out: Optional[bool] = None
        # bf16 products must accumulate in 32-bit all the way
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    def shared_table(self, key, make: Callable[[], torch.Tensor]) -> torch.Tensor:
        """A constant table on the device, built once per distinct key."""
        if key not in self._tables:
            self._tables[key] = make().to(self.device).contiguous()
        return self._tables[key]

    def linear(self, x: torch.Tensor, weight: torch.Tensor,
               bias: Optional[torch.Tensor]) -> torch.Tensor:
        """x @ weight.T (+ bias) in the compute dtype."""
        if self.dtype is torch.float32:
            return ops.gemm_f32(x, weight, bias)
        return F.linear(x, weight, bias)

    def linear_f32_out(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """x @ weight.T with a float32 result (the logits)."""
        if self.dtype is torch.float32:
            return ops.gemm_f32(x, weight, None)
        if self._f32_out is None:
            try:
                torch.mm(x[:1], weight[:8].t(), out_dtype=torch.float32)
                self._f32_out = True
            except (TypeError, RuntimeError):
                self._f32_out = False
        if self._f32_out:
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        return F.linear(x, weight).float()
