#!/usr/bin/env python3
"""Makes the golden outputs in this folder from the reference's own CPU model.

    python tests/golden/make_golden.py --reference /path/to/reference

It compiles, unmodified, the reference's src/model/{model,model_config,safetensors,nn}.cpp,
src/kvcache/{block_manager,paged_kv_cache}.cpp, src/sampler/sampler.cpp,
src/engine/engine.cpp and src/quant/quant.cpp together with ref_dump.cpp (this folder),
against the stand-in for <Eigen/Dense> in eigen_standin/ (Eigen cannot be fetched
offline; only the matrix product goes through the stand-in) and the nlohmann/json.hpp
found in the Python environment.  It then writes a tiny random Qwen2 folder with the
package's random-weights mode into a temporary folder, runs the reference on it and
stores: golden.json (configuration, seed, token ids, checksum of the weights),
forward.f32, chunked.f32 (logits [tokens, vocab], little-endian float32) and greedy.txt.
The model folder itself is not kept: the tests regenerate it from golden.json and check
the checksum.
"""

import argparse
import hashlib
import json
import subprocess
import sys
import sysconfig
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "hidden_size": 48, "num_hidden_layers": 2, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 8, "intermediate_size": 80, "vocab_size": 96,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 64,
}
SEED, STD = 7, 0.08
IDS = [3, 17, 5, 90, 41, 2, 66, 23, 8, 71, 30, 12]
SOURCES = ["src/model/model.cpp", "src/model/model_config.cpp", "src/model/safetensors.cpp",
           "src/model/nn.cpp", "src/kvcache/block_manager.cpp", "src/kvcache/paged_kv_cache.cpp",
           "src/sampler/sampler.cpp", "src/engine/engine.cpp", "src/quant/quant.cpp"]


def find_json_header() -> Path:
    roots = [Path(sysconfig.get_paths()["purelib"]), Path(sys.prefix)]
    for root in roots:
        for hit in root.rglob("nlohmann/json.hpp"):
            return hit.parent.parent
    raise SystemExit("nlohmann/json.hpp not found in the Python environment")


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of the reference project")
    args = parser.parse_args()
    ref = Path(args.reference)
    import torch
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.weights import write_random_model

    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        binary = tmp / "ref_dump"
        cmd = ["g++", "-std=c++20", "-O2", f"-I{ref / 'include'}", f"-I{HERE / 'eigen_standin'}",
               f"-I{find_json_header()}", str(HERE / "ref_dump.cpp"),
               *[str(ref / s) for s in SOURCES], "-o", str(binary)]
        subprocess.run(cmd, check=True)
        model_dir = write_random_model(tmp / "model", config_from_dict(CONFIG), SEED, STD,
                                       torch.bfloat16)
        subprocess.run([str(binary), str(model_dir), str(tmp / "out"), *map(str, IDS)], check=True)
        digest = hashlib.sha256((model_dir / "model.safetensors").read_bytes()).hexdigest()
        for name in ("forward.f32", "chunked.f32", "greedy.txt"):
            (HERE / name).write_bytes((tmp / f"out.{name}").read_bytes())
        (HERE / "golden.json").write_text(json.dumps(
            {"config": CONFIG, "seed": SEED, "std": STD, "dtype": "bfloat16", "ids": IDS,
             "weights_sha256": digest}, indent=2) + "\n")
    print("golden outputs written to", HERE)


if __name__ == "__main__":
    main()
