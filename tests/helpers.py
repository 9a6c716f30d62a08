"""Tiny configurations, model folders and replay helpers shared by the tests."""

from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np
import torch

import plain_qwen2 as plain
from from_scratch_inference_engine_b200.config import config_from_dict
from from_scratch_inference_engine_b200.weights import write_random_model

# Two tiny configurations that differ in every size and option, then two more for the
# window and for a query width that differs from the hidden size.
TINY = {
    "A": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2",
                          num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=16, intermediate_size=176,
                          vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                          tie_word_embeddings=True, max_position_embeddings=128,
                          use_sliding_window=False),
              seed=0, std=0.02),
    "B": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2",
                          num_hidden_layers=3, hidden_size=192, num_attention_heads=6,
                          num_key_value_heads=1, head_dim=32, intermediate_size=512,
                          vocab_size=384, rope_theta=1e6, rms_norm_eps=1e-5,
                          tie_word_embeddings=False, max_position_embeddings=256,
                          use_sliding_window=False),
              seed=1, std=0.05),
    # windowed layers beside a full one, group of 3, width and vocabulary no power of two
    "C": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2",
                          num_hidden_layers=3, hidden_size=120, num_attention_heads=6,
                          num_key_value_heads=2, head_dim=48, intermediate_size=200,
                          vocab_size=331, rope_theta=50000.0, rms_norm_eps=3e-6,
                          tie_word_embeddings=False, max_position_embeddings=512,
                          use_sliding_window=True, sliding_window=21, max_window_layers=1),
              seed=2, std=0.08),
    # explicit head_dim: q width 4 * 32 = 128 differs from hidden 96
    "D": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2",
                          num_hidden_layers=2, hidden_size=96, num_attention_heads=4,
                          num_key_value_heads=4, head_dim=32, intermediate_size=144,
                          vocab_size=200, rope_theta=10000.0, rms_norm_eps=1e-6,
                          tie_word_embeddings=True, max_position_embeddings=256),
              seed=3, std=0.1),
    # head size 64 and pages of 16: prompt portions take the tcgen05 attention kernel
    "E": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2",
                          num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=64, intermediate_size=320,
                          vocab_size=300, rope_theta=10000.0, rms_norm_eps=1e-6,
                          tie_word_embeddings=False, max_position_embeddings=1024),
              seed=5, std=0.05),
    # head size 128, group of 3: decoded tokens can take the tcgen05 attention kernel too
    "F": dict(config=dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2",
                          num_hidden_layers=2, hidden_size=192, num_attention_heads=6,
                          num_key_value_heads=2, head_dim=128, intermediate_size=256,
                          vocab_size=300, rope_theta=100000.0, rms_norm_eps=1e-6,
                          tie_word_embeddings=False, max_position_embeddings=1024),
              seed=6, std=0.05),
}


def make_model_dir(root: Path, name: str) -> Path:
    entry = TINY[name]
    return write_random_model(Path(root) / f"tiny_{name}", config_from_dict(entry["config"]),
                              entry["seed"], entry["std"], torch.bfloat16)


def random_ids(vocab: int, n: int, seed: int) -> List[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


_plain_cache: Dict[Tuple[str, Tuple[int, ...], object], np.ndarray] = {}


def plain_logits(model_dir: Path, ids: List[int], store=None) -> np.ndarray:
    """float64 logits [len(ids), vocab] of the plain implementation (memoised); with
    store=torch.bfloat16, of the plain implementation that writes every operation's result
    in bfloat16 as the engine's bfloat16 path does."""
    key = (str(model_dir), tuple(ids), store)
    if key not in _plain_cache:
        _plain_cache[key] = plain.logits_of(model_dir, ids, store=store).numpy()
    return _plain_cache[key]


# ------------------------------------------------------------------------------ traces
# A trace is a list of steps in the format bin/trace_run reads.
def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    steps = []
    for key, ids in requests.items():
        steps.append({"step": len(steps), "end": [key],
                      "entries": [{"id": key, "tokens": ids, "want": list(range(len(ids)))}]})
    return steps


def trace_tail_by_one(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    steps = []
    for key, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": key, "tokens": ids[:head],
                                   "want": list(range(head))}]})
        for t in range(head, len(ids)):
            steps.append({"step": len(steps), "end": [],
                          "entries": [{"id": key, "tokens": [ids[t]], "want": [0]}]})
        steps[-1]["end"] = [key]
    return steps


def trace_portions(requests: Dict[str, List[int]], seed: int = 0) -> List[dict]:
    rng = random.Random(seed)
    sizes = [7, 2, 13, 2, 5, 3, 16, 2, 9, 4, 31, 2]
    steps = []
    for key, ids in requests.items():
        at = 0
        while at < len(ids):
            n = min(sizes[rng.randrange(len(sizes))], len(ids) - at)
            steps.append({"step": len(steps), "end": [],
                          "entries": [{"id": key, "tokens": ids[at:at + n],
                                       "want": list(range(n))}]})
            at += n
        steps[-1]["end"] = [key]
    return steps


def trace_mixed(requests: Dict[str, List[int]], seed: int = 0, max_live: int = 4,
                decode_tail: int = 6) -> List[dict]:
    """Up to `max_live` live requests; each step holds portions of some beside single
    tokens of others; some requests sit a step out; requests start as others end."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live: Dict[str, int] = {}
    steps = []
    while pending or live:
        while pending and len(live) < max_live and (not live or rng.random() < 0.7):
            key, _ = pending[0]
            pending.pop(0)
            live[key] = 0
        entries, ended = [], []
        for key in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                      # sits this step out
            ids, at = requests[key], live[key]
            left = len(ids) - at
            if left <= decode_tail:
                n = 1
            else:
                n = min(rng.choice([2, 3, 5, 8, 13, 17]), left - decode_tail)
            entries.append({"id": key, "tokens": ids[at:at + n], "want": list(range(n))})
            live[key] = at + n
            if live[key] == len(ids):
                ended.append(key)
                del live[key]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def trace_mixed_with_recompute(requests: Dict[str, List[int]], seed: int = 0, max_live: int = 4,
                               decode_tail: int = 6):
    """The mixed family with preemption as the step function sees it: now and then a live
    request is released in the middle (everything it holds is given back) and fed again
    from position 0 under another name, into pages that others have used meanwhile.
    Returns (steps, requests with the names of the second runs added)."""
    rng = random.Random(seed)
    pending = list(requests.items())
    names = dict(requests)
    live: Dict[str, int] = {}
    released = set()
    steps = []
    while pending or live:
        while pending and len(live) < max_live and (not live or rng.random() < 0.7):
            key, _ = pending.pop(0)
            live[key] = 0
        entries, ended = [], []
        for key in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue
            ids, at = names[key], live[key]
            left = len(ids) - at
            n = 1 if left <= decode_tail else min(rng.choice([2, 3, 5, 8, 13, 17]), left - decode_tail)
            entries.append({"id": key, "tokens": ids[at:at + n], "want": list(range(n))})
            live[key] = at + n
            origin = key.split("~")[0]
            if live[key] == len(ids):
                ended.append(key)
                del live[key]
            elif origin not in released and live[key] >= 9 and rng.random() < 0.3:
                # preempted: released after this step, recomputed later from its first token
                released.add(origin)
                ended.append(key)
                del live[key]
                names[origin + "~again"] = ids
                pending.insert(0, (origin + "~again", ids))
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps, names


def live_tokens_needed(steps: List[dict], round_to: int = 64) -> int:
    """Largest sum over live requests of their token counts, each rounded up to `round_to`."""
    held: Dict[str, int] = {}
    worst = 0
    for step in steps:
        for e in step["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // round_to) * round_to for n in held.values()))
        for key in step["end"]:
            held.pop(key, None)
    return worst


def collect_rows(steps: List[dict], outputs: Dict[int, np.ndarray]):
    """{(request, position): logits row} from per-step outputs [wanted, vocab]."""
    position: Dict[str, int] = {}
    rows = {}
    for step in steps:
        r = 0
        for e in step["entries"]:
            start = position.get(e["id"], 0)
            for w in e["want"]:
                rows[(e["id"], start + w)] = outputs[step["step"]][r]
                r += 1
            position[e["id"]] = start + len(e["tokens"])
    return rows


def run_trace_in_process(runner, steps: List[dict]):
    """Drive a ModelRunner like bin/trace_run does; returns {(request, position): row}."""
    from from_scratch_inference_engine_b200.engine import StepEntry
    live = {}
    outputs = {}
    for step in steps:
        entries = []
        for e in step["entries"]:
            if e["id"] not in live:
                live[e["id"]] = runner.cache.open(e["id"])
            entries.append(StepEntry(live[e["id"]], e["tokens"], e["want"]))
        logits = runner.step(entries)
        if logits is not None:
            outputs[step["step"]] = logits.float().cpu().numpy()
        runner.raise_on_device_error()
        for key in step["end"]:
            runner.cache.close(live.pop(key))
        runner.cache.check()
    return collect_rows(steps, outputs)


OBSERVED: Dict[str, float] = {}      # label -> largest relative difference seen (for reports)


def compare_rows(rows, requests, model_dir, rel: float, label: str = "", store=None):
    """Every row's largest |engine - plain| against rel * max(1, max |plain| of that row).
    Returns (largest difference, largest |plain|, rows beyond the bound); the largest
    difference relative to its row's bound base is kept in OBSERVED[label].  `store`: see
    `plain_logits`."""
    worst, scale, relative = 0.0, 1.0, 0.0
    mismatched = []
    for (key, pos), row in sorted(rows.items()):
        want = plain_logits(model_dir, requests[key], store)[pos]
        base = max(1.0, float(np.abs(want).max()))
        scale = max(scale, base)
        diff = float(np.abs(row.astype(np.float64) - want).max())
        worst = max(worst, diff)
        relative = max(relative, diff / base)
        if diff > rel * base:
            mismatched.append((key, pos, diff))
    if label:
        OBSERVED[label] = max(OBSERVED.get(label, 0.0), relative)
    return worst, scale, mismatched


# ----------------------------------------------------------------- one part on the GPU
class OnePartModel:
    """Stands where a DecoderModel stands in a ModelRunner, but runs a single callable on
    the step's inputs: lets a test step one mixer (or block) through the real cache
    manager, step context and pages without a model around it."""

    def __init__(self, mixer, run, vocab=1 << 20):
        from types import SimpleNamespace
        self.mixer, self.run = mixer, run
        self.schedule = [(0, 0, True)]
        self.spec = SimpleNamespace(vocab_size=vocab, max_position=0)
        self.inputs = None
        self.outputs = None

    def cache_needs(self):
        return [self.mixer.cache_need()]

    def state_needs(self):
        return [self.mixer.state_need()]

    def forward(self, ctx, caches, rows):
        self.outputs = self.run(ctx, self.inputs, caches[0])
        return None
