"""The engine (float32) against the reference's own CPU model and engine, and the test plan's
two workloads as they are written.

tests/golden/<name>/ is a model folder plus what the reference computed from it
(tests/golden/make_golden.py): nothing here goes through the plain implementation except
the temperature workload, which the reference cannot anchor (its requests share one
generator, src/engine/engine.cpp:131-135)."""

import json
from pathlib import Path

import numpy as np
import pytest

import plain_qwen2 as plain
from test_plain import batch_rows, load_case, rows_of

pytestmark = pytest.mark.gpu
CASES = ["A", "B", "G"]


def engine_for(folder, **kwargs):
    from from_scratch_inference_engine_b200 import Engine, LoadedModel
    model = LoadedModel.from_pretrained(folder, dtype="float32", max_positions=1024)
    return Engine(model, **kwargs)


@pytest.mark.parametrize("name", CASES)
def test_whole_sequence_equals_the_reference_forward(name):
    from from_scratch_inference_engine_b200 import LoadedModel
    meta, folder = load_case(name)
    want = rows_of(folder, "forward.f32", meta["config"]["vocab_size"])
    model = LoadedModel.from_pretrained(folder, dtype="float32")
    got = model.forward(meta["scenario"]["ids"]).cpu().numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())
    assert (got.argmax(-1) == want.argmax(-1)).all()


@pytest.mark.parametrize("name", CASES)
def test_mixed_batch_equals_the_reference_forward_batch(name):
    """The reference's forward_batch scenario step for step through the step function: a
    portion beside a whole prompt, then the portion's rest behind cached tokens beside a
    decoded token and a new prompt, then decoded tokens; last-row logits of every item."""
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner, StepEntry
    meta, folder = load_case(name)
    scenario = meta["scenario"]
    want = rows_of(folder, "batch.f32", meta["config"]["vocab_size"])
    model = LoadedModel.from_pretrained(folder, dtype="float32", max_positions=256)
    runner = ModelRunner(model.model, model.runtime, page_size=scenario["block_size"],
                         num_pages=16, max_requests=4)
    handles, got = {}, []
    for step in scenario["batch_steps"]:
        entries = []
        for item in step:
            if item["request"] not in handles:
                handles[item["request"]] = runner.cache.open(item["request"])
            entries.append(StepEntry(handles[item["request"]], item["tokens"],
                                     [len(item["tokens"]) - 1]))
        got.append(runner.step(entries).cpu().numpy().copy())
        runner.raise_on_device_error()
    got = np.concatenate(got)
    assert got.shape == want.shape
    assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())
    assert [handles[k].length for k in "abc"] == [len(batch_rows(scenario)[i]) for i in (5, 3, 6)]


@pytest.mark.parametrize("name", CASES)
def test_concurrent_greedy_requests_equal_the_reference_engine(name):
    """The test plan's workloads: A - prompts of 5/11/17 tokens, 8 greedy tokens, pages of 4;
    B - prompts of 1/7/30/64/100 tokens in portions of 16 beside decoded tokens, pages of 8
    (greedy here; temperature below)."""
    from from_scratch_inference_engine_b200 import SamplingParams
    meta, folder = load_case(name)
    scenario = meta["scenario"]
    want = json.loads((folder / "engine.json").read_text())["greedy"]
    engine = engine_for(folder, block_size=scenario["block_size"], num_blocks=128, max_batch=8,
                        max_step_tokens=16)
    ids = [engine.add_request(p, SamplingParams(temperature=0.0), scenario["greedy_tokens"])
           for p in scenario["greedy_prompts"]]
    engine.run_until_done()
    assert [list(engine.output(i)) for i in ids] == want
    engine.runner.cache.check()
    assert engine.runner.cache.free_pages() == [128]


@pytest.mark.parametrize("pipeline", [False, True])
@pytest.mark.parametrize("name", CASES)
def test_preemption_case_equals_the_reference_engine(name, pipeline):
    """tests/cpp/test_engine.cpp:103-128: two prompts of one block each in a pool of two
    blocks; both need a second block in the same step, one is preempted and recomputed."""
    from from_scratch_inference_engine_b200 import SamplingParams
    meta, folder = load_case(name)
    case = meta["scenario"]["preempt"]
    want = json.loads((folder / "engine.json").read_text())["preempt"]
    engine = engine_for(folder, block_size=meta["scenario"]["block_size"],
                        num_blocks=case["num_blocks"], seed=9, pipeline=pipeline)
    greedy = SamplingParams(temperature=0.0)
    a = engine.add_request(case["a"], greedy, case["tokens"])
    b = engine.add_request(case["b"], greedy, case["tokens"])
    engine.run_until_done()
    assert engine.preemptions() > 0
    assert list(engine.output(a)) == want["a"] and list(engine.output(b)) == want["b"]
    assert engine.runner.cache.free_pages() == [case["num_blocks"]]


def assert_sampled_as_plain(row, params, u, got):
    """`got` is what plain.sample picks from the plain logits `row`, or the uniform number lies
    within 1e-4 of the step of the cumulative distribution between the two tokens (the engine's
    32-bit logits move the steps by about 1e-6)."""
    want = plain.sample(row, params.temperature, params.top_k, params.top_p, u)
    if got == want:
        return
    logits = np.asarray(row, dtype=np.float64)
    order = sorted(range(len(logits)), key=lambda i: (-logits[i], i))
    keep = params.top_k if 0 < params.top_k < len(logits) else len(logits)
    weights = np.exp((logits[order[:keep]] - logits[order[0]]) / params.temperature)
    probs = weights / weights.sum()
    cdf = np.cumsum(probs)
    nucleus = keep if params.top_p >= 1.0 else int(np.searchsorted(cdf, params.top_p) + 1)
    threshold = u * cdf[nucleus - 1]
    at_got, at_want = order.index(got), order.index(want)
    assert at_got < nucleus, f"token {got} lies outside the kept set"
    low, high = sorted((at_got, at_want))
    assert cdf[low] - 1e-4 <= threshold <= cdf[high - 1] + 1e-4 or cdf[high] - cdf[low] < 1e-4, \
        f"engine chose {got}, plain {want}, u = {u}"


def test_temperature_workload_of_the_test_plan_equals_plain_sampling():
    """Config B as the test plan writes its workload: prompts of 1/7/30/64/100 uniform token ids,
    prefilled in portions of 16 beside decoded tokens, pages of 8, 12 tokens each at temperature
    0.8 with a seed.  Every sampled token is re-derived from the plain logits of the request's
    own context and the request's uniform number for that output index."""
    from from_scratch_inference_engine_b200 import SamplingParams
    from from_scratch_inference_engine_b200.sampling.sampler import uniform_draw
    meta, folder = load_case("B")
    prompts = meta["scenario"]["greedy_prompts"]
    assert [len(p) for p in prompts] == [1, 7, 30, 64, 100]
    engine = engine_for(folder, block_size=8, num_blocks=64, max_batch=8, max_step_tokens=16)
    params = [SamplingParams(temperature=0.8, seed=100 + i) for i in range(len(prompts))]
    params[2] = SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=102)
    ids = [engine.add_request(p, q, 12) for p, q in zip(prompts, params)]
    engine.run_until_done()
    config, weights = plain.load(folder)
    outputs = [list(engine.output(i)) for i in ids]
    assert len({tuple(o) for o in outputs}) == len(outputs)
    for prompt, q, out in zip(prompts, params, outputs):
        assert len(out) == 12
        context = list(prompt)
        for index, token in enumerate(out):
            row = plain.forward(config, weights, context)[-1]
            assert_sampled_as_plain(row.tolist(), q, uniform_draw(q.seed, index), token)
            context.append(token)
    # the same requests in a pool so tight that some are preempted and recomputed
    tight = engine_for(folder, block_size=8, num_blocks=16, max_batch=8, max_step_tokens=16)
    ids = [tight.add_request(p, q, 12) for p, q in zip(prompts, params)]
    tight.run_until_done()
    assert tight.preemptions() > 0 and [list(tight.output(i)) for i in ids] == outputs
