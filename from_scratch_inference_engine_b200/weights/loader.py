"""Weights by tensor name, checked against what the model's parts declare.

The check is eager and complete: one `WeightError` lists every missing tensor,
every tensor the model does not use and every wrong shape, instead of the
reference's first-missing-name error (src/cuda/model.cu:740-747) or its lazy
lookup failure (src/model/safetensors.cpp:127-133).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterable, Mapping

import torch

from .safetensors_io import load_file
from .tensor_spec import TensorSpec


class WeightError(RuntimeError):
    pass


def check_tensors(specs: Iterable[TensorSpec], tensors: Mapping[str, torch.Tensor],
                  source: str = "checkpoint") -> None:
    specs = list(specs)
    declared = {}
    for spec in specs:
        if spec.name in declared and declared[spec.name].shape != spec.shape:
            raise WeightError(f"two parts declare '{spec.name}' with different shapes "
                              f"{declared[spec.name].shape} and {spec.shape}")
        declared[spec.name] = spec
    missing = [s.name for s in declared.values() if not s.optional and s.name not in tensors]
    unexpected = [name for name in tensors if name not in declared]
    wrong = []
    for name, spec in declared.items():
        if name in tensors and tuple(tensors[name].shape) != tuple(spec.shape):
            wrong.append(f"{name}: expected {list(spec.shape)}, found "
                         f"{list(tensors[name].shape)}")
    unequal = []
    for name, spec in declared.items():
        if spec.same_as and name in tensors and spec.same_as in tensors and name not in wrong:
            a, b = tensors[name], tensors[spec.same_as]
            if a.shape == b.shape and not torch.equal(a.float(), b.float()):
                unequal.append(f"{name} must equal {spec.same_as} (tied) but differs")
    if missing or unexpected or wrong or unequal:
        lines = [f"{source} does not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(sorted(wrong)))
        if unequal:
            lines.append("  " + "; ".join(unequal))
        raise WeightError("\n".join(lines))


def to_runtime_dtype(tensor: torch.Tensor, spec: TensorSpec, dtype: torch.dtype) -> torch.Tensor:
    """The dtype rule: matrices in the compute dtype, tables int32, 32-bit vectors stay 32-bit."""
    if spec.role == "table":
        return tensor.to(torch.int32)
    if dtype is torch.float32:
        return tensor.to(torch.float32)
    if spec.role == "vector" and tensor.dtype is torch.float32:
        return tensor
    return tensor.to(dtype)


def load_checkpoint(model_dir) -> Dict[str, torch.Tensor]:
    """All tensors of the checkpoint in `model_dir`, in their stored dtypes, on the host:
    `model.safetensors`, or the shards that `model.safetensors.index.json` names (the
    reference reads the single file only, src/model/model.cpp:43-47)."""
    model_dir = Path(model_dir)
    single, index = model_dir / "model.safetensors", model_dir / "model.safetensors.index.json"
    if single.exists() or not index.exists():
        return load_file(single)
    try:
        weight_map = json.loads(index.read_text(encoding="utf-8"))["weight_map"]
    except (OSError, ValueError, KeyError) as error:
        raise WeightError(f"{index} is not a shard index: {error}") from error
    tensors: Dict[str, torch.Tensor] = {}
    for shard in sorted(set(weight_map.values())):
        for name, tensor in load_file(model_dir / shard).items():
            if name in tensors:
                raise WeightError(f"tensor '{name}' is stored in more than one shard")
            tensors[name] = tensor
    absent = sorted(name for name in weight_map if name not in tensors)
    if absent:
        raise WeightError(f"{index} names tensors its shards do not hold: {', '.join(absent)}")
    return tensors
