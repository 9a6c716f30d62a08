"""Reader and writer for the safetensors container, with a hardened header check.

Layout (as the reference parses it, src/model/safetensors.cpp:23-111): 8 bytes of
little-endian header length, a JSON header mapping each tensor name to
{dtype, shape, data_offsets}, then the data region.  Every failure the reference
names is refused here too: a buffer shorter than 8 bytes, a header longer than the
file, invalid JSON, offsets outside the data region, a negative dimension, a byte
count that does not match the shape (checked by division), malformed entries,
overlapping regions and dtypes the engine does not hold.  Tensors are returned
in the dtype they are stored in; widening or narrowing is the loader's business.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Mapping, Tuple

import numpy as np
import torch


class SafeTensorsError(RuntimeError):
    pass


# name in the header -> (numpy dtype used to view the bytes, torch dtype of the result)
_DTYPES = {
    "F32": (np.dtype("<f4"), torch.float32),
    "F16": (np.dtype("<f2"), torch.float16),
    "BF16": (np.dtype("<i2"), torch.bfloat16),
    "I32": (np.dtype("<i4"), torch.int32),
    "I64": (np.dtype("<i8"), torch.int64),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
          torch.int32: "I32", torch.int64: "I64"}


def parse_header(buffer) -> Tuple[Dict[str, dict], int]:
    """Check the container and return ({name: entry}, offset of the data region)."""
    size = len(buffer)
    if size < 8:
        raise SafeTensorsError("safetensors: buffer smaller than the 8-byte header length")
    (header_len,) = struct.unpack("<Q", bytes(buffer[:8]))
    if header_len > size - 8:
        raise SafeTensorsError("safetensors: header length exceeds the buffer")
    try:
        pairs = json.loads(bytes(buffer[8:8 + header_len]).decode("utf-8"),
                           object_pairs_hook=list)
    except (UnicodeDecodeError, json.JSONDecodeError) as error:
        raise SafeTensorsError(f"safetensors: invalid header JSON: {error}") from error
    if not isinstance(pairs, list) or any(not isinstance(p, tuple) for p in pairs):
        raise SafeTensorsError("safetensors: header must be a JSON object")
    region = size - 8 - header_len
    entries: Dict[str, dict] = {}
    spans = []
    for name, meta in pairs:
        if name == "__metadata__":
            continue
        if name in entries:
            raise SafeTensorsError(f"safetensors: duplicate tensor name '{name}'")
        try:
            meta = dict(meta)
            dtype = meta["dtype"]
            shape = list(meta["shape"])
            begin, end = meta["data_offsets"]
            if not isinstance(dtype, str) or any(isinstance(d, bool) or not isinstance(d, int)
                                                 for d in shape + [begin, end]):
                raise TypeError("wrong field types")
        except (KeyError, TypeError, ValueError) as error:
            raise SafeTensorsError(
                f"safetensors: malformed header entry for '{name}': {error}") from error
        if dtype not in _DTYPES:
            raise SafeTensorsError(f"safetensors: unsupported dtype '{dtype}' for {name}")
        if begin < 0 or end < begin or end > region:
            raise SafeTensorsError(f"safetensors: data_offsets out of range for {name}")
        if any(d < 0 for d in shape):
            raise SafeTensorsError(f"safetensors: negative dimension for {name}")
        numel = 1
        for d in shape:
            numel *= d
        item = _DTYPES[dtype][0].itemsize
        nbytes = end - begin
        if nbytes % item != 0 or nbytes // item != numel:
            raise SafeTensorsError(f"safetensors: byte count does not match shape for {name}")
        entries[name] = {"dtype": dtype, "shape": shape, "begin": begin, "end": end}
        if nbytes:
            spans.append((begin, end))
    spans.sort()
    for previous, current in zip(spans, spans[1:]):
        if current[0] < previous[1]:
            raise SafeTensorsError("safetensors: overlapping tensor data regions")
    return entries, 8 + header_len


def parse(buffer) -> Dict[str, torch.Tensor]:
    """All tensors of an in-memory container, each in its stored dtype (a copy)."""
    entries, base = parse_header(buffer)
    raw = np.frombuffer(buffer, dtype=np.uint8)
    out: Dict[str, torch.Tensor] = {}
    for name, entry in entries.items():
        np_dtype, torch_dtype = _DTYPES[entry["dtype"]]
        chunk = raw[base + entry["begin"]: base + entry["end"]]
        array = np.array(chunk, copy=True).view(np_dtype).reshape(entry["shape"])
        tensor = torch.from_numpy(array)
        if torch_dtype is torch.bfloat16:
            tensor = tensor.view(torch.bfloat16)
        out[name] = tensor
    return out


def load_file(path) -> Dict[str, torch.Tensor]:
    path = Path(path)
    try:
        with open(path, "rb") as handle:
            if path.stat().st_size == 0:
                raise SafeTensorsError(
                    "safetensors: buffer smaller than the 8-byte header length")
            with mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ) as mapped:
                return parse(mapped)
    except OSError as error:
        raise SafeTensorsError(f"safetensors: cannot open {path}: {error}") from error


def serialize(tensors: Mapping[str, torch.Tensor]) -> bytes:
    header = {}
    chunks = []
    offset = 0
    for name in sorted(tensors):
        tensor = tensors[name].detach().cpu().contiguous()
        if tensor.dtype not in _NAMES:
            raise SafeTensorsError(f"safetensors: cannot store dtype {tensor.dtype} ({name})")
        if tensor.dtype is torch.bfloat16:
            data = tensor.view(torch.int16).numpy().astype("<i2").tobytes()
        else:
            data = tensor.numpy().astype(_DTYPES[_NAMES[tensor.dtype]][0]).tobytes()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + len(data)]}
        chunks.append(data)
        offset += len(data)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    return struct.pack("<Q", len(text)) + text + b"".join(chunks)


def save_file(tensors: Mapping[str, torch.Tensor], path) -> None:
    Path(path).write_bytes(serialize(tensors))
