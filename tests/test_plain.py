"""The plain implementation against the reference's own CPU model (tests/golden/)."""

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


@pytest.fixture(scope="module")
def golden(tmp_path_factory):
    meta = json.loads((GOLDEN / "golden.json").read_text())
    folder = write_random_model(tmp_path_factory.mktemp("golden_model"),
                                config_from_dict(meta["config"]), meta["seed"], meta["std"],
                                torch.bfloat16)
    digest = hashlib.sha256((folder / "model.safetensors").read_bytes()).hexdigest()
    if digest != meta["weights_sha256"]:
        pytest.skip("the random-weights generator gives other bits on this machine than on "
                    "the one that made the golden files")
    return meta, folder


def test_plain_forward_matches_reference_cpu_model(golden):
    meta, folder = golden
    vocab = meta["config"]["vocab_size"]
    want = np.fromfile(GOLDEN / "forward.f32", dtype="<f4").reshape(-1, vocab)
    got = plain.logits_of(folder, meta["ids"]).numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() < 2e-5
    assert (got.argmax(-1) == want.argmax(-1)).all()


def test_reference_chunked_equals_its_whole_forward(golden):
    meta, _ = golden
    vocab = meta["config"]["vocab_size"]
    whole = np.fromfile(GOLDEN / "forward.f32", dtype="<f4").reshape(-1, vocab)
    chunked = np.fromfile(GOLDEN / "chunked.f32", dtype="<f4").reshape(-1, vocab)
    assert np.abs(whole - chunked).max() < 1e-5


def test_plain_greedy_matches_reference_engine(golden):
    meta, folder = golden
    want = [int(t) for t in (GOLDEN / "greedy.txt").read_text().split()]
    config, weights = plain.load(folder)
    assert plain.greedy_generate(config, weights, meta["ids"], len(want)) == want


def test_plain_window_equals_full_when_window_covers_everything(golden):
    meta, folder = golden
    config, weights = plain.load(folder)
    full = plain.forward(config, weights, meta["ids"])
    config["windows"] = [len(meta["ids"])] * config["layers"]
    assert torch.equal(full, plain.forward(config, weights, meta["ids"]))
    config["windows"] = [3] * config["layers"]
    assert not torch.allclose(full[-1], plain.forward(config, weights, meta["ids"])[-1])


def test_plain_sampler_rules():
    logits = [0.1, 2.0, 2.0, -1.0, 0.5]
    assert plain.sample(logits, 0.0, 0, 1.0, 0.3) == 1            # first maximum
    assert plain.sample(logits, 1.0, 1, 1.0, 0.99) == 1           # top_k = 1 is argmax
    assert plain.sample(logits, 1.0, 0, 1.0, 0.0) == 1
    assert plain.sample(logits, 1.0, 0, 1.0, 0.999999) == 3       # the tail is the smallest
    assert plain.sample([0.0, 10.0, 0.0], 1.0, 0, 0.5, 0.9) == 1  # top_p isolates the peak
