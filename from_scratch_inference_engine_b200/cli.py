"""Command line: generate from a model folder and report timing.

Options follow the reference's harness (benchmarks/harness/bench_engine.py:118-131):
--model-dir (default: environment ENGINE_MODEL_DIR), --num-requests, --prompt,
--max-tokens, --block-size, --num-blocks, --temperature, --json; it submits all requests
up front, drives `Engine.step` and reports TTFT mean/p50/p90, TPOT, tokens/s and
requests/s (bench_engine.py:48-98).  Added: --prompt-ids / --prompt-len (token ids need
no tokenizer), --top-k, --top-p, --seed, --dtype, --max-batch, --max-step-tokens,
--prefix-cache, and --random-weights CONFIG.json with --weights-seed / --std, which
writes a random model folder to --model-dir first.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import statistics
import sys
from pathlib import Path
from time import perf_counter


def _percentile(values, q):
    if not values:
        return 0.0
    ordered = sorted(values)
    return ordered[min(len(ordered) - 1, int(round(q * (len(ordered) - 1))))]


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="generate", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model-dir", default=os.environ.get("ENGINE_MODEL_DIR"))
    parser.add_argument("--num-requests", type=int, default=1)
    parser.add_argument("--prompt", default=None, help="text (needs tokenizer.json in the folder)")
    parser.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    parser.add_argument("--prompt-len", type=int, default=0, help="uniform random ids of this length")
    parser.add_argument("--max-tokens", type=int, default=64)
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-blocks", type=int, default=4096)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--max-batch", type=int, default=256)
    parser.add_argument("--max-step-tokens", type=int, default=2048)
    parser.add_argument("--prefix-cache", type=int, default=1, choices=[0, 1])
    parser.add_argument("--random-weights", default=None, metavar="CONFIG.json")
    parser.add_argument("--weights-seed", type=int, default=0)
    parser.add_argument("--std", type=float, default=0.02)
    parser.add_argument("--json", action="store_true", help="emit metrics as JSON")
    args = parser.parse_args(argv)
    if not args.model_dir:
        parser.error("--model-dir (or ENGINE_MODEL_DIR) is required")

    from . import LLM, SamplingParams, SeqStatus, write_random_model
    from .config import config_from_dict

    if args.random_weights:
        config = config_from_dict(json.loads(Path(args.random_weights).read_text()))
        write_random_model(args.model_dir, config, args.weights_seed, args.std)
    llm = LLM(args.model_dir, block_size=args.block_size, num_blocks=args.num_blocks,
              seed=args.seed, max_batch=args.max_batch, dtype=args.dtype,
              enable_prefix_cache=bool(args.prefix_cache), max_step_tokens=args.max_step_tokens)
    vocab = llm.model.model.spec.vocab_size
    if args.prompt_ids:
        prompts = [[int(t) for t in args.prompt_ids.split(",")]] * args.num_requests
    elif args.prompt_len > 0:
        rng = random.Random(args.seed)
        prompts = [[rng.randrange(vocab) for _ in range(args.prompt_len)]
                   for _ in range(args.num_requests)]
    elif args.prompt is not None:
        prompts = [llm.tokenizer.encode(args.prompt).ids] * args.num_requests
    else:
        parser.error("one of --prompt, --prompt-ids, --prompt-len is required")

    engine = llm.engine
    params = SamplingParams(args.temperature, args.top_k, args.top_p)
    start = perf_counter()
    ids = [engine.add_request(list(p), params, args.max_tokens, llm.eos_id) for p in prompts]
    first, finished = {}, {}
    while engine.has_work():
        if engine.step() == 0:
            raise RuntimeError("no request can make progress")
        now = perf_counter()
        for rid in ids:
            if rid not in first and engine.output(rid):
                first[rid] = now
            if rid not in finished and engine.status(rid) is SeqStatus.Finished:
                finished[rid] = now
    wall = perf_counter() - start
    outputs = [list(engine.output(rid)) for rid in ids]
    ttft = [(first[r] - start) * 1000.0 for r in ids if r in first]
    tpot = [(finished[r] - first[r]) * 1000.0 / (len(engine.output(r)) - 1)
            for r in ids if r in finished and len(engine.output(r)) > 1]
    total = sum(len(o) for o in outputs)
    report = {
        "requests": len(ids), "prompt_tokens": len(prompts[0]), "max_tokens": args.max_tokens,
        "total_output_tokens": total, "wall_seconds": wall,
        "throughput_tokens_per_s": total / wall if wall > 0 else 0.0,
        "requests_per_s": len(ids) / wall if wall > 0 else 0.0,
        "ttft_ms_mean": statistics.fmean(ttft) if ttft else 0.0,
        "ttft_ms_p50": _percentile(ttft, 0.5), "ttft_ms_p90": _percentile(ttft, 0.9),
        "tpot_ms_mean": statistics.fmean(tpot) if tpot else 0.0,
        "engine": engine.stats(), "outputs": outputs,
    }
    if args.json:
        print(json.dumps(report, indent=2))
    else:
        print(f"requests:              {report['requests']}")
        print(f"prompt tokens (each):  {report['prompt_tokens']}")
        print(f"max tokens:            {report['max_tokens']}")
        print(f"output tokens (total): {total}")
        print(f"wall time:             {wall:.3f} s")
        print(f"throughput:            {report['throughput_tokens_per_s']:.1f} tok/s")
        print(f"requests/s:            {report['requests_per_s']:.2f}")
        print(f"TTFT mean/p50/p90:     {report['ttft_ms_mean']:.1f} / {report['ttft_ms_p50']:.1f} "
              f"/ {report['ttft_ms_p90']:.1f} ms")
        print(f"TPOT mean:             {report['tpot_ms_mean']:.1f} ms")
        print(f"preemptions / prefix hits: {engine.preemptions()} / {engine.prefix_hits()}")
        for rid, out in zip(ids, outputs):
            text = ""
            if args.prompt is not None:
                text = "  " + repr(llm.tokenizer.decode(out))
            print(f"[{rid}] {','.join(map(str, out))}{text}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
