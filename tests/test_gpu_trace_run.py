"""bin/trace_run as a user runs it: a subprocess, steps on standard input, logits in files."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import helpers
from helpers import TINY

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def replay(folder, dtype, steps, out_dir, max_tokens, *options):
    text = "".join(json.dumps(step) + "\n" for step in steps)
    done = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
                           dtype, "--out", str(out_dir), "--max-tokens", str(max_tokens), *options],
                          input=text, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done ")] == \
        [f"done {s['step']}" for s in steps]
    return done


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_mixed_trace(tmp_path, dtype):
    folder = helpers.make_model_dir(tmp_path, "B")
    vocab = TINY["B"]["config"]["vocab_size"]
    requests = {key: helpers.random_ids(vocab, n, i)
                for i, (key, n) in enumerate({"a": 90, "b": 40, "c": 70, "d": 33, "e": 64}.items())}
    steps = helpers.trace_mixed(requests, seed=3)
    steps.append({"step": len(steps), "entries": [], "end": []})          # an empty step
    steps.append({"step": len(steps), "end": ["z"],
                  "entries": [{"id": "z", "tokens": requests["a"][:9], "want": []}]})
    need = helpers.live_tokens_needed(steps, round_to=64)
    out = tmp_path / "out"
    replay(folder, dtype, steps, out, need)
    vocab_rows = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        path = out / f"{step['step']}.f32"
        if wanted == 0:
            assert not path.exists()
            continue
        data = np.fromfile(path, dtype="<f4")
        assert data.size == wanted * vocab
        vocab_rows[step["step"]] = data.reshape(wanted, vocab)
    rows = helpers.collect_rows(steps, vocab_rows)
    worst, scale, bad = helpers.compare_rows(rows, requests, folder,
                                             1e-4 if dtype == "float32" else 4e-2)
    assert not bad, f"worst {worst:.3e} at scale {scale:.3f}: {bad[:3]}"


def test_trace_run_with_other_pages_and_fewer_live_requests(tmp_path):
    """--page-size and --max-live: pages of 8 tokens, four requests live at most, and a
    request released in the middle that runs again from its first token."""
    folder = helpers.make_model_dir(tmp_path, "D")
    vocab = TINY["D"]["config"]["vocab_size"]
    requests = {key: helpers.random_ids(vocab, n, i)
                for i, (key, n) in enumerate({"a": 70, "b": 35, "c": 48, "d": 20, "e": 9}.items())}
    steps, names = helpers.trace_mixed_with_recompute(requests, seed=4, max_live=4)
    need = helpers.live_tokens_needed(steps, round_to=64)
    out = tmp_path / "out"
    replay(folder, "float32", steps, out, need, "--page-size", "8", "--max-live", "4")
    outputs = {step["step"]: np.fromfile(out / f"{step['step']}.f32", dtype="<f4").reshape(-1, vocab)
               for step in steps}
    rows = helpers.collect_rows(steps, outputs)
    worst, scale, bad = helpers.compare_rows(rows, names, folder, 1e-4)
    assert not bad, f"worst {worst:.3e} at scale {scale:.3f}: {bad[:3]}"
    # a fifth live request is refused
    crowd = [{"step": 0, "end": [], "entries": [{"id": str(k), "tokens": [1, 2], "want": []}
                                                 for k in range(5)]}]
    done = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
                           "float32", "--out", str(tmp_path / "o2"), "--max-tokens", "512",
                           "--max-live", "4"], input=json.dumps(crowd[0]) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert done.returncode != 0


def test_trace_run_reports_bad_input(tmp_path):
    folder = helpers.make_model_dir(tmp_path, "A")
    step = {"step": 0, "entries": [{"id": "a", "tokens": [1, 999], "want": [0]}], "end": []}
    done = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
                           "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                          input=json.dumps(step) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert done.returncode != 0 and "out of range" in done.stderr
