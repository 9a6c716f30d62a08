#!/usr/bin/env python3
"""Parity of the engine with the plain implementation at the Qwen2.5-7B layer sizes.

    python tests/parity_7b_shape.py [--layers 28] [--dtype float32]

Not collected by pytest (it needs ~100 GB of GPU memory and a minute): random bf16
weights N(0, 0.02) at the 7B shape are drawn once on the GPU and given both to the engine
(float32 path by default) and to the plain implementation (tests/plain_qwen2.py, float64,
on the GPU).  Three requests of 72, 48 and 33 tokens are replayed whole, with the last 32
tokens one by one, in portions of changing size and mixed, through a page pool that holds
just what the live requests need.  Prints one JSON line with the largest |engine - plain|
per way of cutting, the largest |plain logit| and whether every argmax agrees.
"""

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
sys.path.insert(0, str(HERE.parent))

import helpers  # noqa: E402
import plain_qwen2 as plain  # noqa: E402


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--layers", type=int, default=28)
    parser.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    parser.add_argument("--decode-tcgen05", action="store_true",
                        help="bfloat16: decoded tokens take the tcgen05 attention kernel that the engine "
                             "otherwise keeps for large batches")
    args = parser.parse_args()
    sys.path.insert(0, str(HERE.parent))
    import bench
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.engine import LoadedModel, ModelRunner
    from from_scratch_inference_engine_b200.parts import tensor_specs

    shape = dict(bench.SHAPE_7B)
    shape["num_hidden_layers"] = args.layers
    config = config_from_dict(shape)
    generator = torch.Generator(device="cuda").manual_seed(0)
    tensors = {}
    for spec in tensor_specs(config.build_spec()):
        if spec.optional:
            continue
        values = torch.randn(spec.shape, generator=generator, device="cuda") * 0.02
        if spec.init == "gain":
            values += 1.0
        tensors[spec.name] = values.to(torch.bfloat16)
    requests = {key: helpers.random_ids(config.vocab_size, n, seed)
                for seed, (key, n) in enumerate({"a": 72, "b": 48, "c": 33}.items())}

    plain_config = plain.read_config_dict(shape)
    want = {}
    for key, ids in requests.items():          # one layer's weights in float64 at a time
        class Widening(dict):
            def __getitem__(self, name):
                return tensors[name].double()

            def __contains__(self, name):
                return name in tensors
        want[key] = plain.forward(plain_config, Widening(), ids).cpu().numpy()
    scale = max(float(np.abs(w).max()) for w in want.values())

    options = {"decode_tcgen05_min_blocks": 1} if args.decode_tcgen05 else {}
    model = LoadedModel.from_tensors(config, tensors, dtype=args.dtype, max_positions=512, **options)
    result = {"layers": args.layers, "dtype": args.dtype, "max_abs_plain_logit": scale,
              "decode_tcgen05": bool(args.decode_tcgen05)}
    families = {"whole": helpers.trace_whole(requests),
                "tail_by_one": helpers.trace_tail_by_one(requests),
                "portions": helpers.trace_portions(requests, 5),
                "mixed": helpers.trace_mixed(requests, 5)}
    for name, steps in families.items():
        need = helpers.live_tokens_needed(steps, round_to=16)
        runner = ModelRunner(model.model, model.runtime, page_size=16, num_pages=need // 16,
                             max_requests=4)
        rows = helpers.run_trace_in_process(runner, steps)
        worst, agree = 0.0, True
        for (key, pos), row in rows.items():
            worst = max(worst, float(np.abs(row - want[key][pos]).max()))
            agree = agree and int(row.argmax()) == int(want[key][pos].argmax())
        result[name] = {"max_abs_diff": worst, "rel": worst / max(1.0, scale),
                        "argmax_agree": agree, "steps": len(steps), "pool_tokens": need}
        del runner
    print(json.dumps(result))


if __name__ == "__main__":
    main()
