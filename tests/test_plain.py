"""The plain implementation against the reference's own CPU model and engine.

tests/golden/<name>/ holds, for the two tiny configurations of the test plan (A, B) and a
third with a head size of 8 (G), a model folder and what the reference made of it
(tests/golden/make_golden.py): logits of a whole sequence, of a portion followed by single
tokens, of a mixed batch over one block pool, and tokens of its engine - several requests at
once, and two requests in a pool of two blocks, where one is preempted and recomputed."""

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from from_scratch_inference_engine_b200.config import config_from_dict
from from_scratch_inference_engine_b200.weights import write_random_model

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = ["A", "B", "G"]


def load_case(name):
    folder = GOLDEN / name
    meta = json.loads((folder / "golden.json").read_text())
    digest = hashlib.sha256((folder / "model.safetensors").read_bytes()).hexdigest()
    assert digest == meta["weights_sha256"], "the golden model file is not the one the outputs were made from"
    return meta, folder


def rows_of(folder, kind, vocab):
    return np.fromfile(folder / kind, dtype="<f4").reshape(-1, vocab)


@pytest.mark.parametrize("name", CASES)
def test_plain_forward_matches_reference_cpu_model(name):
    meta, folder = load_case(name)
    want = rows_of(folder, "forward.f32", meta["config"]["vocab_size"])
    got = plain.logits_of(folder, meta["scenario"]["ids"]).numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() < 2e-5
    assert (got.argmax(-1) == want.argmax(-1)).all()


@pytest.mark.parametrize("name", CASES)
def test_reference_chunked_equals_its_whole_forward(name):
    meta, folder = load_case(name)
    vocab = meta["config"]["vocab_size"]
    assert np.abs(rows_of(folder, "forward.f32", vocab) - rows_of(folder, "chunked.f32", vocab)).max() < 1e-5


def batch_rows(scenario):
    """(tokens of the request up to and including the item) for every item of every step, in
    the order the reference's forward_batch returned its last-row logits."""
    fed, out = {}, []
    for step in scenario["batch_steps"]:
        for item in step:
            fed[item["request"]] = fed.get(item["request"], []) + item["tokens"]
            out.append(list(fed[item["request"]]))
    return out


@pytest.mark.parametrize("name", CASES)
def test_plain_matches_reference_mixed_batch(name):
    """Portions behind cached tokens, decoded tokens and whole prompts in one batch
    (Model::forward_batch): the last row of every item equals the plain whole forward."""
    meta, folder = load_case(name)
    want = rows_of(folder, "batch.f32", meta["config"]["vocab_size"])
    contexts = batch_rows(meta["scenario"])
    assert len(contexts) == len(want) == 7
    for tokens, row in zip(contexts, want):
        got = plain.logits_of(folder, tokens)[-1].numpy()
        assert np.abs(got - row).max() < 2e-5


@pytest.mark.parametrize("name", CASES)
def test_plain_greedy_matches_reference_engine(name):
    meta, folder = load_case(name)
    engine = json.loads((folder / "engine.json").read_text())
    config, weights = plain.load(folder)
    scenario = meta["scenario"]
    for prompt, want in zip(scenario["greedy_prompts"], engine["greedy"]):
        if len(prompt) > 40:
            continue          # the long prompts are for the GPU engine; 64-bit Python loops are slow
        assert plain.greedy_generate(config, weights, prompt, len(want)) == want


@pytest.mark.parametrize("name", CASES)
def test_reference_preemption_case(name):
    """tests/cpp/test_engine.cpp:103-128 on this model: the pool forced a preemption and the
    tokens are those of each request alone; the plain implementation gives the same."""
    meta, folder = load_case(name)
    record = json.loads((folder / "engine.json").read_text())["preempt"]
    assert record["preemptions"] > 0
    assert record["a"] == record["alone_a"] and record["b"] == record["alone_b"]
    config, weights = plain.load(folder)
    case = meta["scenario"]["preempt"]
    assert plain.greedy_generate(config, weights, case["a"], case["tokens"]) == record["a"]
    assert plain.greedy_generate(config, weights, case["b"], case["tokens"]) == record["b"]


@pytest.mark.parametrize("name", CASES)
def test_random_weights_mode_reproduces_the_golden_model(name, tmp_path):
    """The generator is keyed by (seed, tensor name, element index): the same bits everywhere."""
    meta, folder = load_case(name)
    made = write_random_model(tmp_path / "again", config_from_dict(meta["config"]), meta["seed"],
                              meta["std"], torch.bfloat16)
    digest = hashlib.sha256((made / "model.safetensors").read_bytes()).hexdigest()
    assert digest == meta["weights_sha256"]


def test_plain_window_equals_full_when_window_covers_everything():
    meta, folder = load_case("G")
    ids = meta["scenario"]["ids"]
    config, weights = plain.load(folder)
    full = plain.forward(config, weights, ids)
    config["windows"] = [len(ids)] * config["layers"]
    assert torch.equal(full, plain.forward(config, weights, ids))
    config["windows"] = [3] * config["layers"]
    assert not torch.allclose(full[-1], plain.forward(config, weights, ids)[-1])


def test_plain_sampler_rules():
    logits = [0.1, 2.0, 2.0, -1.0, 0.5]
    assert plain.sample(logits, 0.0, 0, 1.0, 0.3) == 1            # first maximum
    assert plain.sample(logits, 1.0, 1, 1.0, 0.99) == 1           # top_k = 1 is argmax
    assert plain.sample(logits, 1.0, 0, 1.0, 0.0) == 1
    assert plain.sample(logits, 1.0, 0, 1.0, 0.999999) == 3       # the tail is the smallest
    assert plain.sample([0.0, 10.0, 0.0], 1.0, 0, 0.5, 0.9) == 1  # top_p isolates the peak
