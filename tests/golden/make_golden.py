#!/usr/bin/env python3
"""Makes the golden outputs in this folder from the reference's own CPU model and engine.

    python tests/golden/make_golden.py --reference /path/to/reference

It compiles, unmodified, the reference's src/model/{model,model_config,safetensors,nn}.cpp,
src/kvcache/{block_manager,paged_kv_cache}.cpp, src/sampler/sampler.cpp,
src/engine/engine.cpp and src/quant/quant.cpp together with ref_dump.cpp (this folder),
against the stand-in for <Eigen/Dense> in eigen_standin/ (Eigen cannot be fetched
offline; only the matrix product goes through the stand-in) and the nlohmann/json.hpp
found in the Python environment.  For each configuration below (the two tiny
configurations of the test plan, which differ in every size and option, and a third with a
head size of 8) it writes a random model folder with the package's random-weights mode,
runs the reference on it and stores, under <name>/: golden.json (configuration, seed,
scenario, checksum of the weights), model.safetensors (the weights themselves, so that
the comparison does not depend on the generator giving the same bits everywhere),
forward.f32, chunked.f32, batch.f32 (little-endian float32 rows of `vocab` logits) and
engine.json (tokens of the reference's engine).
"""

import argparse
import hashlib
import json
import random
import shutil
import subprocess
import sys
import sysconfig
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))


def qwen2(**sizes):
    base = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2"}
    base.update(sizes)
    return base


CASES = {
    # the two tiny configurations of the test plan: they differ in every size and option
    "A": dict(config=qwen2(num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=16, intermediate_size=176,
                           vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                           tie_word_embeddings=True, max_position_embeddings=128,
                           use_sliding_window=False),
              seed=0, std=0.02, block_size=4, tokens=17, greedy_prompts=[5, 11, 17],
              greedy_tokens=8),
    "B": dict(config=qwen2(num_hidden_layers=3, hidden_size=192, num_attention_heads=6,
                           num_key_value_heads=1, head_dim=32, intermediate_size=512,
                           vocab_size=384, rope_theta=1e6, rms_norm_eps=1e-5,
                           tie_word_embeddings=False, max_position_embeddings=256,
                           use_sliding_window=False),
              seed=1, std=0.05, block_size=8, tokens=30, greedy_prompts=[1, 7, 30, 64, 100],
              greedy_tokens=12),
    # head size 8, query width 48 = hidden, tied head
    "G": dict(config=qwen2(hidden_size=48, num_hidden_layers=2, num_attention_heads=6,
                           num_key_value_heads=2, head_dim=8, intermediate_size=80, vocab_size=96,
                           rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                           max_position_embeddings=64),
              seed=7, std=0.08, block_size=4, tokens=12, greedy_prompts=[12], greedy_tokens=8),
}
SOURCES = ["src/model/model.cpp", "src/model/model_config.cpp", "src/model/safetensors.cpp",
           "src/model/nn.cpp", "src/kvcache/block_manager.cpp", "src/kvcache/paged_kv_cache.cpp",
           "src/sampler/sampler.cpp", "src/engine/engine.cpp", "src/quant/quant.cpp"]


def find_json_header() -> Path:
    roots = [Path(sysconfig.get_paths()["purelib"]), Path(sys.prefix)]
    for root in roots:
        for hit in root.rglob("nlohmann/json.hpp"):
            return hit.parent.parent
    raise SystemExit("nlohmann/json.hpp not found in the Python environment")


def scenario_for(name: str, case: dict) -> dict:
    rng = random.Random(sum(map(ord, name)))
    vocab = case["config"]["vocab_size"]
    ids = [rng.randrange(vocab) for _ in range(case["tokens"])]
    a, b, c = ids[:9], ids[3:8], ids[5:12]
    extra = [rng.randrange(vocab) for _ in range(3)]
    # step 1: a portion of a beside all of b; step 2: the rest of a (behind cached tokens),
    # one decoded token of b, all of c; step 3: decoded tokens of a and c
    batch_steps = [
        [{"request": "a", "tokens": a[:6]}, {"request": "b", "tokens": b}],
        [{"request": "a", "tokens": a[6:]}, {"request": "b", "tokens": [extra[0]]},
         {"request": "c", "tokens": c}],
        [{"request": "a", "tokens": [extra[1]]}, {"request": "c", "tokens": [extra[2]]}],
    ]
    block = case["block_size"]
    return {"ids": ids, "block_size": block, "batch_steps": batch_steps,
            "greedy_prompts": [[rng.randrange(vocab) for _ in range(n)]
                               for n in case["greedy_prompts"]],
            "greedy_tokens": case["greedy_tokens"],
            # each prompt fills one block; both need a second one in the same step of a pool
            # that has none left
            "preempt": {"a": [rng.randrange(vocab) for _ in range(block)],
                        "b": [rng.randrange(vocab) for _ in range(block)],
                        "tokens": 4, "num_blocks": 2}}


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
        for name, case in CASES.items():
            model_dir = write_random_model(tmp / f"model_{name}", config_from_dict(case["config"]),
                                           case["seed"], case["std"], torch.bfloat16)
            scenario = scenario_for(name, case)
            (tmp / "scenario.json").write_text(json.dumps(scenario))
            subprocess.run([str(binary), str(model_dir), str(tmp / "scenario.json"),
                            str(tmp / "out")], check=True)
            target = HERE / name
            target.mkdir(exist_ok=True)
            for kind in ("forward.f32", "chunked.f32", "batch.f32", "engine.json"):
                shutil.copyfile(tmp / f"out.{kind}", target / kind)
            shutil.copyfile(model_dir / "model.safetensors", target / "model.safetensors")
            shutil.copyfile(model_dir / "config.json", target / "config.json")
            digest = hashlib.sha256((model_dir / "model.safetensors").read_bytes()).hexdigest()
            (target / "golden.json").write_text(json.dumps(
                {"config": case["config"], "seed": case["seed"], "std": case["std"],
                 "dtype": "bfloat16", "scenario": scenario, "weights_sha256": digest},
                indent=1) + "\n")
            print("golden outputs written to", target)


if __name__ == "__main__":
    main()
