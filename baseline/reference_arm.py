"""The bench's reference arm: the unmodified reference engine on the same shape and workload.

Nothing of this repository's package is imported here.  A model folder with random bfloat16
weights of the wanted shape is written with plain torch (config.json with the reference's
keys, model.safetensors in the safetensors layout), the binary that
baseline/build_reference.py builds from the reference's own sources is run on it, and its
figures come back as a dictionary.  The reference widens every tensor to float32 at load and
computes in float32 (strict-IEEE cuBLAS SGEMM, 64-bit softmax: src/cuda/device.cu:139-190,
322-357): it has no other precision, so the arm's dtype is fp32.
"""

from __future__ import annotations

import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent


def tensor_shapes(shape: dict):
    """(name, shape, kind) of every tensor of a Qwen2 checkpoint, in file order."""
    h, inter, vocab = shape["hidden_size"], shape["intermediate_size"], shape["vocab_size"]
    q = shape["num_attention_heads"] * shape["head_dim"]
    kv = shape["num_key_value_heads"] * shape["head_dim"]
    yield "model.embed_tokens.weight", (vocab, h), "matrix"
    for layer in range(shape["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        yield p + "input_layernorm.weight", (h,), "gain"
        for name, rows in (("q", q), ("k", kv), ("v", kv)):
            yield p + f"self_attn.{name}_proj.weight", (rows, h), "matrix"
            yield p + f"self_attn.{name}_proj.bias", (rows,), "matrix"
        yield p + "self_attn.o_proj.weight", (h, q), "matrix"
        yield p + "post_attention_layernorm.weight", (h,), "gain"
        yield p + "mlp.gate_proj.weight", (inter, h), "matrix"
        yield p + "mlp.up_proj.weight", (inter, h), "matrix"
        yield p + "mlp.down_proj.weight", (h, inter), "matrix"
    yield "model.norm.weight", (h,), "gain"
    if not shape.get("tie_word_embeddings", False):
        yield "lm_head.weight", (vocab, h), "matrix"


def write_model_folder(folder: Path, shape: dict, seed: int = 0, std: float = 0.02) -> int:
    """config.json + model.safetensors (BF16) with N(0, std) matrices and biases and gains of
    1 + N(0, std); returns the bytes written."""
    import torch
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(shape, indent=1))
    entries, header, offset = list(tensor_shapes(shape)), {}, 0
    for name, dims, _ in entries:
        count = 1
        for d in dims:
            count *= d
        header[name] = {"dtype": "BF16", "shape": list(dims), "data_offsets": [offset, offset + 2 * count]}
        offset += 2 * count
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    generator = torch.Generator(device=device).manual_seed(seed)
    with open(folder / "model.safetensors", "wb") as out:
        out.write(struct.pack("<Q", len(text)))
        out.write(text)
        for name, dims, kind in entries:
            values = torch.randn(dims, generator=generator, device=device, dtype=torch.float32) * std
            if kind == "gain":
                values += 1.0
            out.write(values.to(torch.bfloat16).cpu().view(torch.int16).numpy().tobytes())
    return offset + 8 + len(text)


def run(shape: dict, batch: int, context: int, steps: int, warmup: int, prefill_tokens: int,
        timeout_s: float = 3000.0) -> dict:
    """Figures of the reference binary, or {"unavailable": reason}."""
    sys.path.insert(0, str(HERE))
    try:
        import build_reference
        binary = build_reference.build(verbose=False)
    except (SystemExit, subprocess.CalledProcessError, OSError) as error:
        return {"unavailable": f"the reference's CUDA engine could not be built here: {error}"}
    finally:
        sys.path.pop(0)
    h, inter = shape["hidden_size"], shape["intermediate_size"]
    bytes_needed = sum(2 * int(__import__("math").prod(d)) for _, d, _ in tensor_shapes(shape))
    root = Path(os.environ.get("TMPDIR", tempfile.gettempdir()))
    if shutil.disk_usage(root).free < bytes_needed * 1.05:
        return {"unavailable": f"no room for the {bytes_needed / 1e9:.1f} GB model folder the "
                               f"reference loads under {root}"}
    folder = Path(tempfile.mkdtemp(prefix="fsie_reference_model_", dir=root))
    try:
        write_model_folder(folder, shape)
        print(f"reference arm: model folder written ({bytes_needed / 1e9:.1f} GB), running "
              f"{binary.name}", file=sys.stderr, flush=True)
        done = subprocess.run([str(binary), str(folder), str(batch), str(context), str(steps),
                               str(warmup), str(prefill_tokens)], capture_output=True, text=True,
                              timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference did not finish inside {timeout_s:.0f} s"}
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    sys.stderr.write(done.stderr[-2000:])
    if done.returncode != 0:
        last = (done.stderr.strip().splitlines() or ["no message"])[-1]
        return {"unavailable": f"the reference binary exited with {done.returncode}: {last}"}
    return json.loads(done.stdout.strip().splitlines()[-1])
