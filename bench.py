#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen2.5-7B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl engine|reference]

A step is one decode step of a batch of 8 requests whose contexts end at 4,096 tokens
(random bf16 weights, uniform random token ids).  One JSON line comes out:

  value     decoded tokens per second, timed on the device with CUDA events over K steps
            of the step function with device-side argmax (no host round trip inside)
  e2e       the same through the Python entry point (`Engine.step`): every step copies
            its inputs from pinned host memory and reads the chosen tokens back
  prefill   one 2,048-token prompt through the step function: tokens/s, ms and the
            fraction of the measured bf16 matrix peak; `points`: four such prompts in one
            step, and one prompt in portions of 512 tokens
  roofline  bytes the decode step must read (every weight once + the live requests'
            keys and values) / its time, against the measured copy bandwidth
  points    decode tokens/s at batch 1 and 64 (32 timed steps or more)
  decode_by_context  the headline batch with contexts ending at 2,048 / 3,072 / 4,096 tokens
  fp32      the true 32-bit path of the same model (own FFMA products, float32 cache): decode
            tokens/s with its HBM fraction (28 GB of weights per step) and the prefill of one
            prompt against the nominal FFMA peak

Between timed steps nothing flushes L2: every step streams 15 GB of weights, far more
than the 126 MB of L2.  `--impl reference` runs the same shape and workload through the
unmodified reference engine (its CUDA path compiled from its own sources by
baseline/build_reference.py, since its CMake build needs the network) and prints the same
line with "impl": "reference"; where that build is impossible it prints an `unavailable`
line and exits 0.  This engine runs on one GPU only: --gpus N > 1 exits 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPE_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28,
                hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                intermediate_size=18944, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
                tie_word_embeddings=False, max_position_embeddings=32768,
                use_sliding_window=False)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# FFMA peak of the float32 path (no tensor-core mode): 148 SMs x 128 lanes x 2 flop x 1.965 GHz,
# nominal; the measured-peaks file has no float32 figure
FP32_FFMA_TFLOPS = 74.4


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    source = "fallback"
    values = dict(FALLBACK_PEAKS)
    if path.exists():
        try:
            data = json.loads(path.read_text())
            found = 0
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                value = data.get(key) if isinstance(data, dict) else None
                if isinstance(value, dict):        # a record with the figure inside
                    value = next((value[k] for k in ("value", "median", "mean") if k in value), None)
                if isinstance(value, (int, float)) and value > 0:
                    values[key] = float(value)
                    found += 1
            if found:
                source = "measured"
        except (OSError, ValueError, TypeError):
            pass
    return values, source


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.process, self.thread = [], None, None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            self.samples.append([field.strip() for field in line.split(",")])

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, reasons, max_mhz = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for sample in self.samples:
            if len(sample) < 7:
                continue
            try:
                clocks.append(float(sample[0]))
                max_mhz = float(sample[1])
            except ValueError:
                continue
            for name, field in zip(names, sample[3:7]):
                if field.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_mhz,
                "reasons": sorted(reasons), "samples": len(clocks)}


def weight_bytes(config, layers):
    h, i = config.hidden_size, config.intermediate_size
    per_layer = (config.q_width + 2 * config.kv_width) * h + h * config.q_width + 3 * i * h
    return 2 * (layers * per_layer + config.vocab_size * h)


def kv_bytes_per_token(config, layers):
    return 2 * 2 * config.kv_width * layers


def prefill_flops(config, layers, tokens):
    h, i = config.hidden_size, config.intermediate_size
    per_layer = (config.q_width + 2 * config.kv_width) * h + h * config.q_width + 3 * i * h
    linear = 2.0 * tokens * (layers * per_layer + config.vocab_size * h / tokens)   # head: 1 row
    attention = layers * 4.0 * config.q_width * tokens * (tokens + 1) / 2           # causal half
    return linear + attention


SHAPE_1P5B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=28,
                  hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                  intermediate_size=8960, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                  tie_word_embeddings=True, max_position_embeddings=32768, use_sliding_window=False)
SHAPE_14B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=48,
                 hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                 intermediate_size=13824, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
                 tie_word_embeddings=False, max_position_embeddings=32768, use_sliding_window=False)


def serving_workload(args) -> int:
    """Continuous batching at the Qwen2.5-1.5B shape: 256 requests, prompts of 64-2,048 uniform
    token ids, 32-512 output tokens, half of them behind one common 512-token prefix, all
    submitted up front.  Prints one JSON line: total tokens/s, time to first token and per
    output token, preemptions, prefix hits."""
    import numpy as np
    import torch
    from from_scratch_inference_engine_b200 import Engine, LoadedModel, SamplingParams, SeqStatus
    from from_scratch_inference_engine_b200.config import config_from_dict

    config = config_from_dict(dict(SHAPE_1P5B))
    rng = np.random.default_rng(1)
    requests = args.requests
    model = LoadedModel.from_random(config, seed=0, std=0.02, dtype="bfloat16", max_positions=4096)
    engine = Engine(model, block_size=16, num_blocks=args.num_blocks, max_batch=256,
                    enable_prefix_cache=True, max_step_tokens=args.step_tokens)
    prefix = rng.integers(0, config.vocab_size, size=512).tolist()
    prompts, outputs = [], []
    for r in range(requests):
        length = int(rng.integers(64, 2049))
        body = rng.integers(0, config.vocab_size, size=length).tolist()
        prompts.append((prefix + body)[:max(length, 513)] if r % 2 == 0 else body)
        outputs.append(int(rng.integers(32, 513)))
    # as a server does at start-up: kernels compiled and decode graphs captured before requests come
    engine.generate(prompts[0][:40], SamplingParams(temperature=0.0), max_tokens=4)
    graphs = engine.warm_up(2048 + 512)
    torch.cuda.synchronize()
    start = time.perf_counter()
    ids = [engine.add_request(p, SamplingParams(temperature=0.0), max_tokens=n)
           for p, n in zip(prompts, outputs)]
    first, done = {}, {}
    silent, live = set(ids), set(ids)          # no token seen yet; not finished yet
    while engine.has_work():
        if engine.step() == 0:
            raise RuntimeError("no request can make progress")
        now = time.perf_counter()
        for rid in [r for r in silent if engine.output(r)]:
            first[rid] = now
            silent.discard(rid)
        for rid in [r for r in live if engine.status(r) is SeqStatus.Finished]:
            done[rid] = now
            live.discard(rid)
    torch.cuda.synchronize()
    wall = time.perf_counter() - start
    produced = sum(len(engine.output(r)) for r in ids)
    ttft = sorted((first[r] - start) * 1000.0 for r in ids)
    tpot = [(done[r] - first[r]) * 1000.0 / (len(engine.output(r)) - 1) for r in ids
            if len(engine.output(r)) > 1]
    stats = engine.stats()
    print(json.dumps({
        "metric": "continuous batching tokens/s (Qwen2.5-1.5B shape, 256 requests)", "impl": "engine",
        "value": (sum(map(len, prompts)) + produced) / wall, "unit": "tokens/s", "n_gpus": 1,
        "output_tokens_per_s": produced / wall, "wall_s": wall, "requests": requests,
        "prompt_tokens": sum(map(len, prompts)), "output_tokens": produced,
        "ttft_ms": {"mean": statistics.fmean(ttft), "p50": ttft[len(ttft) // 2],
                    "p90": ttft[int(len(ttft) * 0.9)]},
        "tpot_ms_mean": statistics.fmean(tpot), "steps": stats["steps"],
        "preemptions": stats["preemptions"], "prefix_hits": stats["prefix_hits"], "graphs_captured_before": graphs,
        "num_blocks": args.num_blocks, "dtype": "bf16",
        "data": "synthetic: random bf16 weights, uniform random token ids"}))
    return 0


def long_context_workload(args) -> int:
    """The Qwen2.5-14B shape on one GPU: decode at batch 32 with contexts of 8,192 tokens, and
    chunked prefill (2,048-token portions) of an 8,192-token prompt.  One JSON line."""
    import numpy as np
    import torch
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner, StepEntry
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.kernels import ops

    shape = dict(SHAPE_14B)
    layers = args.layers or shape["num_hidden_layers"]
    shape["num_hidden_layers"] = layers
    config = config_from_dict(shape)
    peak, peak_source = peaks()
    batch, context, portion, page = 32, 8192, 2048, 16
    steps, warmup = min(args.steps, 32), max(args.warmup, 3)
    rng = np.random.default_rng(0)
    model = LoadedModel.from_random(config, seed=0, std=0.02, dtype="bfloat16", max_positions=context + 64,
                                    **({"share_tiles": False} if args.share_tiles == "off" else {}))
    device = model.runtime.device

    def timed(fn):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end)

    # ---- chunked prefill of one prompt (the second run is timed: kernels are compiled by the first)
    runner = ModelRunner(model.model, model.runtime, page_size=page, num_pages=2 * (context // page + 1),
                         max_requests=2)
    prompt = rng.integers(0, config.vocab_size, size=context).tolist()
    portions_ms = []
    for attempt in range(2):
        handle = runner.cache.open(("p", attempt))
        portions_ms = [timed(lambda at=at: runner.step([StepEntry(handle, prompt[at:at + portion],
                                                                  [portion - 1] if at + portion == context else [])]))
                       for at in range(0, context, portion)]
        runner.cache.close(handle)
    runner.raise_on_device_error()
    del runner
    torch.cuda.empty_cache()
    prefill_ms = sum(portions_ms)
    flops = prefill_flops(config, layers, context)

    # ---- decode at batch 32: contexts are reserved, not computed (the cache holds zeros; the
    # kernels read and multiply them all the same)
    runner = ModelRunner(model.model, model.runtime, page_size=page,
                         num_pages=batch * (context // page + 1), max_requests=batch)
    start_len = context - (steps + warmup)
    handles = []
    for r in range(batch):
        handle = runner.cache.open(r)
        runner.cache.reserve(handle, start_len)
        runner.cache.commit(handle, start_len)
        handles.append(handle)
    tokens = rng.integers(0, config.vocab_size, size=(steps + warmup, batch))
    picks = torch.empty(batch, dtype=torch.int32, device=device)

    def step(index):
        logits = runner.step([StepEntry(h, [int(tokens[index, b])], [0]) for b, h in enumerate(handles)])
        ops.argmax(logits, picks)
    for index in range(warmup):
        step(index)
    clocks = ClockSampler()
    clocks.start()
    ms_step = timed(lambda: [step(warmup + index) for index in range(steps)]) / steps
    clock_record = clocks.stop()
    runner.raise_on_device_error()
    read_bytes = weight_bytes(config, layers) + batch * (context - steps / 2) * kv_bytes_per_token(config, layers)
    print(json.dumps({
        "metric": "decode tok/s @ batch 32, context 8,192; chunked prefill of 8,192 tokens (Qwen2.5-14B shape)",
        "impl": "engine", "value": batch * 1000.0 / ms_step, "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_step, "dtype": "bf16",
        "roofline": {"bound": "hbm", "achieved": read_bytes / (ms_step * 1e-3) / 1e9, "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": read_bytes / (ms_step * 1e-3) / 1e9 / peak["hbm_gbs"],
                     "peaks": peak_source},
        "prefill": {"value": context * 1000.0 / prefill_ms, "tokens": context, "ms": prefill_ms,
                    "portion_ms": [round(m, 2) for m in portions_ms],
                    "frac": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12)},
        "config": {"model": "Qwen2.5-14B shape", "layers": layers, "layers_of_shape": SHAPE_14B["num_hidden_layers"],
                   "global_batch": batch, "seq_len": context, "prefill_portion": portion, "kv_page": page},
        "clocks": clock_record,
        "data": "synthetic: random bf16 weights N(0,0.02), uniform random token ids; decode contexts reserved, not computed"}))
    return 0


def timeline_workload(args) -> int:
    """Where the time of one decode step goes while it runs as it does in serving (a replayed
    graph whose kernels overlap their heads and tails): kernel start and end times of one
    step as the profiling interface records them, per kernel kind what its end adds to
    the latest end before it, and one layer in order.  Text, not a bench value."""
    import numpy as np
    import torch
    from torch.profiler import ProfilerActivity, profile
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner, StepEntry
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.kernels import ops

    shape = dict(SHAPE_7B)
    shape["num_hidden_layers"] = args.layers or shape["num_hidden_layers"]
    config = config_from_dict(shape)
    batch, context, page = args.batch, args.context, 16
    model = LoadedModel.from_random(config, seed=0, std=0.02, dtype="bfloat16", max_positions=context + 64,
                                    **({"share_tiles": False} if args.share_tiles == "off" else {}))
    rng = np.random.default_rng(0)
    runner = ModelRunner(model.model, model.runtime, page_size=page,
                         num_pages=batch * (context // page + 2), max_requests=batch)
    handles = []
    for r in range(batch):
        handle = runner.cache.open(r)
        ids = rng.integers(0, config.vocab_size, size=context - 40).tolist()
        for at in range(0, len(ids), 2048):
            runner.step([StepEntry(handle, ids[at:at + 2048])])
        handles.append(handle)
    picks = torch.empty(batch, dtype=torch.int32, device=model.runtime.device)
    if args.timeline_of == "prefill":
        # one prompt of --prefill-tokens in one step, again and again
        for handle in handles:
            runner.cache.close(handle)
        prompt = rng.integers(0, config.vocab_size, size=args.prefill_tokens).tolist()

        def step():
            handle = runner.cache.open("p")
            runner.step([StepEntry(handle, prompt, [len(prompt) - 1])])
            runner.cache.close(handle)
    else:
        def step():
            logits = runner.step([StepEntry(h, [int(rng.integers(0, 1000))], [0]) for h in handles])
            ops.argmax(logits, picks)
    for _ in range(8):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(6):
            step()
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
    first = [i for i, e in enumerate(events) if "embed" in e.name]
    if len(first) < 5:
        print("timeline: the steps were not found in the profile")
        return 1
    one = events[first[3]:first[4]]
    origin = one[0].time_range.start
    name = lambda e: e.name.replace("fsie::", "").replace("void ", "")[:44]
    what = f"prefill step of {args.prefill_tokens} tokens" if args.timeline_of == "prefill" else \
        f"decode step, batch {batch}, context {context}"
    print(f"{what}, {shape['num_hidden_layers']} layers: "
          f"{events[first[4]].time_range.start - origin:.1f} us, {len(one)} kernels")
    print("   start     end  kernel (us from the step's first kernel; the second layer and what follows it)")
    per_layer = max(1, (len(one) - 5) // shape["num_hidden_layers"])
    for e in one[2 + per_layer:2 + 2 * per_layer + 2]:
        print(f"{e.time_range.start - origin:8.1f} {e.time_range.end - origin:7.1f}  {name(e)}")
    # every kernel waits for the one before it, so the step advances with the latest end so far:
    # a kernel's share is what its end adds to that
    cost, count, latest = {}, {}, origin
    for e in one:
        cost[name(e)] = cost.get(name(e), 0.0) + max(0.0, e.time_range.end - latest)
        count[name(e)] = count.get(name(e), 0) + 1
        latest = max(latest, e.time_range.end)
    print("what each kernel's end adds to the latest end before it, summed over the step:")
    for key, value in sorted(cost.items(), key=lambda kv: -kv[1]):
        print(f"{value:9.1f} us  x{count[key]:3d}  {key}")
    return 0


def reference_arm(args) -> int:
    """The same metric and shape through the unmodified reference engine (built from its own
    sources by baseline/build_reference.py; its CUDA engine, CudaEngine::step, decodes the batch
    and reads the chosen tokens back every step).  Nothing of this package runs on this arm."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm as arm
    shape = dict(SHAPE_7B)
    full_layers = shape["num_hidden_layers"]
    layers = args.layers or full_layers
    shape["num_hidden_layers"] = layers
    steps, warmup = args.steps, max(args.warmup, 3)
    clocks = ClockSampler()
    clocks.start()
    figures = arm.run(shape, args.batch, args.context, steps, warmup, args.prefill_tokens)
    clock_record = clocks.stop()
    if "unavailable" in figures:
        print(json.dumps({"impl": "reference", "unavailable": figures["unavailable"]}))
        return 0
    value = figures["decode_tokens_per_s"]
    record = {
        "metric": "decode tok/s @ batch 8, context 4,096 (Qwen2.5-7B shape)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": figures["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic: random bf16 weights N(0,0.02) widened to fp32 by the reference's "
                "loader, uniform token ids",
        "impl": "reference",
        "config": {"model": "Qwen2.5-7B shape", "global_batch": args.batch,
                   "seq_len": args.context, "parallelism": "single GPU", "layers": layers,
                   "layers_of_shape": full_layers, "hidden": shape["hidden_size"],
                   "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"],
                   "vocab": shape["vocab_size"], "prefill_tokens": args.prefill_tokens,
                   "precision": "fp32 only: the reference has no other",
                   "timing": "wall clock around CudaEngine::step, which synchronises the device "
                             "and reads the tokens back every step",
                   "l2": "not flushed: each step streams 30 GB of weights, L2 is 126 MB"},
        # the reference engine has one way to step: ids and positions go to the device and the
        # chosen tokens come back every step, so the figure above already is end to end
        "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": figures["ms_per_step"],
                "h2d_bytes_per_step": 16.0 * args.batch, "d2h_bytes_per_step": 8.0 * args.batch},
        "prefill": {"value": (args.prefill_tokens * 1000.0 / figures["prefill_ms"]
                              if figures["prefill_ms"] > 0 else None),
                    "tokens": args.prefill_tokens, "ms": figures["prefill_ms"]},
        "load_s": figures["load_s"], "fill_s": figures["fill_s"],
        "clocks": clock_record,
    }
    print(json.dumps(record))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None,
                        help="timed decode steps (default 64; with --impl reference 8: a step of the "
                             "reference engine takes about 11 s)")
    parser.add_argument("--warmup", type=int, default=None, help="untimed steps before them (default 8; reference 3)")
    parser.add_argument("--impl", default="engine", choices=["engine", "reference"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has")
    parser.add_argument("--prefill-tokens", type=int, default=2048)
    parser.add_argument("--points", default="1,64", help="extra decode batch sizes ('' = none)")
    parser.add_argument("--contexts", default="2048,3072,4096",
                        help="contexts at which decoding at --batch is also timed ('' = none)")
    parser.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "fp32", "float32"],
                        help="compute dtype of the whole run (the default run adds a short fp32 section)")
    parser.add_argument("--few-token-limit", type=int, default=0,
                        help="steps of up to this many tokens take the engine's few-token tcgen05 product "
                             "(0 = the engine's choice, 32; up to 64 for measuring that choice)")
    parser.add_argument("--timeline-of", default="decode", choices=["decode", "prefill"],
                        help="timeline: a decode step, or a step of one prompt of --prefill-tokens")
    parser.add_argument("--share-tiles", default="on", choices=["on", "off"],
                        help="off: the tiled product leaves a partial last round of tiles to the pairs of "
                             "blocks it falls to instead of sharing it out among all (for measuring that choice)")
    parser.add_argument("--fp32-steps", type=int, default=8,
                        help="decode steps timed on the float32 path after the bf16 run (0 = skip)")
    parser.add_argument("--workload", default="decode", choices=["decode", "serving", "long", "timeline"],
                        help="decode: the default measurement; serving: continuous batching of 256 "
                             "requests at the 1.5B shape; long: the 14B shape, decode at batch 32 with "
                             "8,192-token contexts and chunked prefill of an 8,192-token prompt; "
                             "timeline: kernel start and end times inside one decode step (text)")
    parser.add_argument("--requests", type=int, default=256)
    parser.add_argument("--step-tokens", type=int, default=2048, help="serving: token budget of one step")
    parser.add_argument("--num-blocks", type=int, default=16384)
    args = parser.parse_args()
    if args.steps is None:
        args.steps = 8 if args.impl == "reference" else 64
    if args.warmup is None:
        args.warmup = 3 if args.impl == "reference" else 8

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload == "serving":
        return serving_workload(args)
    if args.workload == "long":
        return long_context_workload(args)
    if args.workload == "timeline":
        return timeline_workload(args)

    import numpy as np
    import torch
    from from_scratch_inference_engine_b200 import (Engine, LoadedModel, ModelRunner,
                                                    SamplingParams, StepEntry)
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.kernels import ops

    shape = dict(SHAPE_7B)
    full_layers = shape["num_hidden_layers"]
    layers = args.layers or full_layers
    shape["num_hidden_layers"] = layers
    config = config_from_dict(shape)
    peak, peak_source = peaks()
    steps, warmup = args.steps, max(args.warmup, 3)
    page = 16
    rng = np.random.default_rng(0)
    compute = "bfloat16" if args.dtype in ("bf16", "bfloat16") else "float32"
    bytes_per = 2 if compute == "bfloat16" else 4
    options = {"few_token_limit": args.few_token_limit} if args.few_token_limit else {}
    if args.share_tiles == "off":
        options["share_tiles"] = False
    model = LoadedModel.from_random(config, seed=0, std=0.02, dtype=compute,
                                    max_positions=args.context + 64, **options)
    device = model.runtime.device

    def timed(fn, count):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for index in range(count):
            fn(index)
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / count          # ms per call

    def fill(runner, batch, length):
        """Prefill `batch` requests of `length` tokens through the step function."""
        handles = []
        for r in range(batch):
            handle = runner.cache.open(r)
            ids = rng.integers(0, config.vocab_size, size=length).tolist()
            for at in range(0, length, 2048):
                runner.step([StepEntry(handle, ids[at:at + 2048])])
            handles.append(handle)
        return handles

    def decode_rate(use_model, batch, count, warm, context_end):
        """Device-timed decode: `count` steps of `batch` single tokens with device argmax, the
        last of which brings the contexts to `context_end` tokens.  (ms per step, launches)"""
        start_len = context_end - (count + warm)
        pages = batch * (-(-context_end // page) + 1)
        runner = ModelRunner(use_model.model, use_model.runtime, page_size=page, num_pages=pages,
                             max_requests=batch)
        handles = fill(runner, batch, start_len)
        tokens = rng.integers(0, config.vocab_size, size=(count + warm, batch))
        picks = torch.empty(batch, dtype=torch.int32, device=device)

        def step(index):
            logits = runner.step([StepEntry(h, [int(tokens[index, b])], [0])
                                  for b, h in enumerate(handles)])
            ops.argmax(logits, picks)
        for index in range(warm):
            step(index)
        before = ops.launches
        ms = timed(lambda index: step(warm + index), count)
        launches = ops.launches - before
        runner.raise_on_device_error()
        del runner
        torch.cuda.empty_cache()
        return ms, launches

    def step_bytes(batch, context_mid, element_bytes):
        """What a decode step has to read: every weight once and the live requests' keys and values."""
        return (weight_bytes(config, layers) + batch * context_mid * kv_bytes_per_token(config, layers)) \
            * element_bytes / 2

    def prefill_figures(use_model, tokens, repeat=3):
        """One prompt whole, four prompts in one step, and one prompt in portions of 512 tokens."""
        runner = ModelRunner(use_model.model, use_model.runtime, page_size=page,
                             num_pages=4 * (tokens // page + 1), max_requests=4,
                             max_step_tokens=4 * tokens)
        prompts = [rng.integers(0, config.vocab_size, size=tokens).tolist() for _ in range(4)]

        def whole(index):
            handle = runner.cache.open(("p", index))
            runner.step([StepEntry(handle, prompts[index % 4], [tokens - 1])])
            runner.cache.close(handle)

        def four(index):
            handles = [runner.cache.open(("f", index, r)) for r in range(4)]
            runner.step([StepEntry(h, prompts[r], [tokens - 1]) for r, h in enumerate(handles)])
            for handle in handles:
                runner.cache.close(handle)

        def portions(index):
            handle = runner.cache.open(("c", index))
            for at in range(0, tokens, 512):
                last = at + 512 >= tokens
                runner.step([StepEntry(handle, prompts[index % 4][at:at + 512],
                                       [len(prompts[index % 4][at:at + 512]) - 1] if last else [])])
            runner.cache.close(handle)
        out = {}
        for name, fn, count in (("whole", whole, tokens), ("x4", four, 4 * tokens),
                                ("portions_512", portions, tokens)):
            fn(0)
            out[name] = (min(timed(fn, 1) for _ in range(repeat)), count)
        runner.raise_on_device_error()
        del runner
        torch.cuda.empty_cache()
        return out

    clocks = ClockSampler()
    clocks.start()
    ms_step, launches = decode_rate(model, args.batch, steps, warmup, args.context)
    clock_record = clocks.stop()
    value = args.batch * 1000.0 / ms_step

    # ---- end to end through the Python entry point
    slack = 64           # requests that finish their prompt early decode while others prefill
    start_len = args.context - (steps + warmup + slack) - 1
    engine = Engine(model, block_size=page, num_blocks=args.batch * (-(-args.context // page) + 1),
                    max_batch=args.batch, max_step_tokens=2048)
    for _ in range(args.batch):
        engine.add_request(rng.integers(0, config.vocab_size, size=start_len).tolist(),
                           SamplingParams(temperature=0.0),
                           max_tokens=steps + warmup + slack + 1)
    while not all(seq.prefilled for seq in engine.scheduler.sequences.values()):
        engine.step()
    for _ in range(warmup):
        engine.step()
    ring, sampler = engine.runner._ring, engine.sampler
    h2d0, d2h0 = ring.bytes_staged + sampler.bytes_to_device, sampler.bytes_to_host
    # The engine overlaps its steps: one is always in flight.  The clock starts after the step
    # that the warm-up left in flight has completed, and stops when the last of the K steps
    # launched inside the region has completed: exactly K steps, each with its copy of inputs
    # from pinned memory and its read of the chosen tokens, the first of them launched onto an
    # idle GPU.  The slower of the host's clock and the device's events counts.
    torch.cuda.synchronize()
    wall = time.perf_counter()
    ms_e2e = timed(lambda index: engine.step(), steps)
    wall = (time.perf_counter() - wall) * 1000.0 / steps
    ms_e2e = max(ms_e2e, wall)
    h2d = (ring.bytes_staged + sampler.bytes_to_device - h2d0) / steps
    d2h = (sampler.bytes_to_host - d2h0) / steps
    del engine
    torch.cuda.empty_cache()

    # ---- prefill: one prompt whole (the headline), four in one step, one in portions of 512
    tokens = args.prefill_tokens
    matrix_peak = peak["bf16_tflops"] * 1e12 if compute == "bfloat16" else FP32_FFMA_TFLOPS * 1e12
    flops = prefill_flops(config, layers, tokens)
    figures = prefill_figures(model, tokens, repeat=3 if compute == "bfloat16" else 1)
    ms_prefill = figures["whole"][0]
    prefill_record = {"value": tokens * 1000.0 / ms_prefill, "tokens": tokens, "ms": ms_prefill,
                      "frac": flops / (ms_prefill * 1e-3) / matrix_peak,
                      "points": {name: {"tokens_per_s": count * 1000.0 / ms, "ms": ms}
                                 for name, (ms, count) in figures.items() if name != "whole"}}

    # ---- roofline of the decode step
    achieved = step_bytes(args.batch, args.context - (steps + 1) / 2, bytes_per) / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peak["hbm_gbs"], "peaks": peak_source}

    # ---- further decode points: other batch sizes at the same context, and this batch size at
    # contexts of 2,048 and 3,072 tokens (the headline's contexts end at --context)
    points, by_context = {}, {}
    count = max(32, steps) if compute == "bfloat16" else max(8, steps // 4)
    for batch in [int(b) for b in args.points.split(",") if b]:
        ms, _ = decode_rate(model, batch, count, max(3, warmup), args.context)
        points[f"decode_b{batch}"] = batch * 1000.0 / ms
    for context_end in [int(c) for c in args.contexts.split(",") if c]:
        if context_end == args.context:
            ms = ms_step
        else:
            ms, _ = decode_rate(model, args.batch, count, max(3, warmup), context_end)
        got = step_bytes(args.batch, context_end - (count + 1) / 2, bytes_per) / (ms * 1e-3) / 1e9
        by_context[str(context_end)] = {"tokens_per_s": args.batch * 1000.0 / ms,
                                        "hbm_frac": got / peak["hbm_gbs"]}
    if by_context:
        by_context["mean_tokens_per_s"] = statistics.fmean(v["tokens_per_s"] for v in by_context.values())

    # ---- the float32 path (own FFMA products, float32 cache): a few steps, one prompt
    fp32_record = None
    if compute == "bfloat16" and args.fp32_steps > 0:
        del model
        torch.cuda.empty_cache()
        model32 = LoadedModel.from_random(config, seed=0, std=0.02, dtype="float32",
                                          max_positions=args.context + 64)
        ms32, _ = decode_rate(model32, args.batch, args.fp32_steps, 3, args.context)
        got32 = step_bytes(args.batch, args.context - (args.fp32_steps + 1) / 2, 4) / (ms32 * 1e-3) / 1e9
        fig32 = prefill_figures(model32, tokens, repeat=1)
        fp32_record = {"decode_tokens_per_s": args.batch * 1000.0 / ms32, "ms_per_step": ms32,
                       "steps": args.fp32_steps, "hbm_gbs": got32, "hbm_frac": got32 / peak["hbm_gbs"],
                       "prefill_ms": fig32["whole"][0],
                       "prefill_tokens_per_s": tokens * 1000.0 / fig32["whole"][0],
                       "prefill_frac_of_ffma_peak": flops / (fig32["whole"][0] * 1e-3) / (FP32_FFMA_TFLOPS * 1e12),
                       "ffma_peak_tflops": FP32_FFMA_TFLOPS}
        del model32
        torch.cuda.empty_cache()

    record = {
        "metric": f"decode tok/s @ batch {args.batch}, context {args.context:,} (Qwen2.5-7B shape)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if compute == "bfloat16" else "fp32",
        "data": "synthetic: random bf16 weights N(0,0.02), uniform random token ids",
        "impl": "engine",
        "config": {"model": "Qwen2.5-7B shape", "global_batch": args.batch,
                   "seq_len": args.context, "parallelism": "single GPU", "layers": layers,
                   "layers_of_shape": full_layers, "hidden": config.hidden_size,
                   "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                   "head_dim": config.head_dim, "intermediate": config.intermediate_size,
                   "vocab": config.vocab_size, "kv_page": page,
                   "prefill_tokens": tokens,
                   "l2": "not flushed: each step streams 15 GB of weights, L2 is 126 MB"},
        "e2e": {"value": args.batch * 1000.0 / ms_e2e, "unit": "tokens/s",
                "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": prefill_record,
        "roofline": roofline,
        "points": points,
        "decode_by_context": by_context,
        "clocks": clock_record,
    }
    if fp32_record is not None:
        record["fp32"] = fp32_record
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
