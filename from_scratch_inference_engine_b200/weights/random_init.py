"""Random-weights mode: a model folder from a configuration and a seed.

Every value is a function of (seed, tensor name, element index) only, so the
same folder comes out on every machine and in every order of creation.  The
reference's fixture draws N(0, 0.02) for every tensor including gains
(tests/cpp/tiny_model.hpp:46-73); here gains are 1 + N(0, std), which keeps the
norms near identity at any depth.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Iterable

import numpy as np
import torch

from .safetensors_io import save_file
from .tensor_spec import TensorSpec

_MASK = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix(x: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser on uint64 arrays."""
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _MASK
    x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _MASK
    x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _MASK
    return x ^ (x >> np.uint64(31))


def standard_normal(seed: int, name: str, count: int) -> np.ndarray:
    """`count` N(0,1) draws keyed by (seed, name), as float64 (Box-Muller on hashed counters)."""
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    key = np.uint64(int.from_bytes(digest[:8], "little"))
    with np.errstate(over="ignore"):
        counters = np.arange(count, dtype=np.uint64)
        a = _mix(counters * np.uint64(2) + key)
        b = _mix(counters * np.uint64(2) + np.uint64(1) + key)
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740993.0   # (0, 1)
    u2 = (b >> np.uint64(11)).astype(np.float64) / 9007199254740992.0           # [0, 1)
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def random_tensor(spec: TensorSpec, seed: int, std: float, dtype: torch.dtype) -> torch.Tensor:
    count = int(np.prod(spec.shape)) if spec.shape else 1
    if spec.role == "table":
        raise ValueError(f"no random recipe for integer table {spec.name}")
    if spec.init == "zeros":
        values = np.zeros(count)
    elif spec.init == "ones":
        values = np.ones(count)
    elif spec.init == "gain":
        values = 1.0 + std * standard_normal(seed, spec.name, count)
    elif spec.init == "normal":
        values = std * standard_normal(seed, spec.name, count)
    else:
        raise ValueError(f"unknown init '{spec.init}' for {spec.name}")
    tensor = torch.from_numpy(values.astype(np.float32)).reshape(spec.shape)
    return tensor.to(dtype)


def random_tensors(specs: Iterable[TensorSpec], seed: int, std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.optional or spec.name in out:
            continue
        out[spec.name] = random_tensor(spec, seed, std, dtype)
    return out


def random_tensors_on_device(specs: Iterable[TensorSpec], seed: int, std: float = 0.02,
                             device="cuda:0", dtype: torch.dtype = torch.bfloat16
                             ) -> Dict[str, torch.Tensor]:
    """The same recipe (matrices and biases N(0, std), gains 1 + N(0, std), rounded to `dtype`)
    drawn by the device's own generator, for sizes at which hashing billions of counters on the
    host would take minutes: benchmarks and tests at real layer sizes.  Reproducible on one
    kind of device for one seed, but not the bits of `random_tensors`."""
    generator = torch.Generator(device=device).manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.optional or spec.name in out:
            continue
        if spec.role == "table":
            raise ValueError(f"no random recipe for integer table {spec.name}")
        if spec.init in ("zeros", "ones"):
            values = torch.full(spec.shape, float(spec.init == "ones"), device=device)
        elif spec.init in ("gain", "normal"):
            values = torch.randn(spec.shape, generator=generator, device=device,
                                 dtype=torch.float32) * std
            if spec.init == "gain":
                values += 1.0
        else:
            raise ValueError(f"unknown init '{spec.init}' for {spec.name}")
        out[spec.name] = values.to(dtype)
    return out


def write_random_model(model_dir, config, seed: int, std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write config.json and model.safetensors for `config` with weights drawn from `seed`."""
    from ..parts.model import tensor_specs   # late: parts import weights

    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    data = config.to_dict()
    data["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                           torch.float16: "float16"}[dtype]
    (model_dir / "config.json").write_text(json.dumps(data, indent=2) + "\n", encoding="utf-8")
    tensors = random_tensors(tensor_specs(config.build_spec()), seed, std, dtype)
    save_file(tensors, model_dir / "model.safetensors")
    return model_dir
