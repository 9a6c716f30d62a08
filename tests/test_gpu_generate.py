"""Generation through the Python entry point and the engine's scheduling on the GPU
(reference behaviour: tests/cpp/test_engine.cpp:38-162, tests/cpp/test_cuda_engine.cpp:45-79)."""

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain
from helpers import TINY

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model_dir(root, name) for name in ("A", "B", "C")}


def assert_greedy_agrees(folder, prompt, got, gap_allowed):
    """Token for token, or up to a first difference that is a near tie of the plain logits."""
    config, weights = plain.load(folder)
    ids = list(prompt)
    for index, token in enumerate(got):
        row = plain.forward(config, weights, ids)[-1]
        want = plain.sample(row, 0.0, 0, 1.0, 0.0)
        if token != want:
            gap = float(row[want] - row[token])
            assert gap <= gap_allowed * max(1.0, float(row.abs().max())), \
                f"token {index}: engine chose {token}, plain {want}, gap {gap:.3e}"
            return index
        ids.append(token)
    return len(got)


@pytest.mark.parametrize("name,block_size", [("A", 4), ("B", 8)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_llm(folders, name, block_size, dtype):
    from from_scratch_inference_engine_b200 import LLM, GenerationConfig
    llm = LLM(folders[name], block_size=block_size, num_blocks=64, dtype=dtype, max_batch=4,
              eos_id=-1)
    vocab = TINY[name]["config"]["vocab_size"]
    for n, seed in ((5, 1), (17, 2), (1, 3)):
        prompt = helpers.random_ids(vocab, n, seed)
        out = llm.generate_ids(prompt, GenerationConfig(max_tokens=8))
        assert len(out) == 8
        agreed = assert_greedy_agrees(folders[name], prompt, out,
                                      1e-5 if dtype == "float32" else 2e-2)
        if dtype == "float32":
            assert agreed == 8
    llm.engine.runner.cache.check()
    assert llm.engine.runner.cache.free_pages() == [64]


def test_model_forward_entry_point(folders):
    from from_scratch_inference_engine_b200 import LoadedModel
    model = LoadedModel.from_pretrained(folders["B"], dtype="float32")
    ids = helpers.random_ids(384, 21, 4)
    got = model.forward(ids).cpu().numpy()
    want = helpers.plain_logits(folders["B"], ids)
    assert got.shape == want.shape and np.abs(got - want).max() < 1e-4
    with pytest.raises(IndexError):
        model.forward([1, 2, 384])


def engine_for(folder, dtype="float32", **kwargs):
    from from_scratch_inference_engine_b200 import Engine, LoadedModel
    options = dict(block_size=4, num_blocks=64, seed=0, max_batch=8, max_step_tokens=16)
    options.update(kwargs)
    blocks = options["num_blocks"]
    blocks = max(blocks) if isinstance(blocks, list) else blocks
    model = LoadedModel.from_pretrained(folder, dtype=dtype,
                                        max_positions=options["block_size"] * blocks)
    return Engine(model, **options)


def test_two_concurrent_requests_equal_each_alone(folders):
    from from_scratch_inference_engine_b200 import SamplingParams
    greedy = SamplingParams(temperature=0.0)
    p1, p2 = helpers.random_ids(256, 11, 1), helpers.random_ids(256, 23, 2)
    alone = [engine_for(folders["A"]).generate(p, greedy, 10) for p in (p1, p2)]
    engine = engine_for(folders["A"])
    a = engine.add_request(p1, greedy, 10)
    b = engine.add_request(p2, greedy, 10)
    engine.run_until_done()
    assert engine.output(a) == alone[0] and engine.output(b) == alone[1]
    assert engine.stats()["tokens_prefilled"] == 34


def same_or_near_tie(folder, prompts, outputs, want, dtype):
    """float32: the tokens are the expected ones.  bfloat16: another batch may round otherwise
    (other key splits, another product kernel), so each request's tokens must agree with the
    plain implementation up to a first difference that is a near tie of the plain logits."""
    if dtype == "float32":
        assert outputs == want
        return
    for prompt, out, expected in zip(prompts, outputs, want):
        assert len(out) == len(expected)
        assert_greedy_agrees(folder, prompt, out, 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_run_out_preemption_recomputes_to_the_same_tokens(folders, dtype):
    from from_scratch_inference_engine_b200 import SamplingParams
    greedy = SamplingParams(temperature=0.0)
    prompts = [helpers.random_ids(384, 5, s) for s in (5, 6)]
    alone = [engine_for(folders["B"], dtype, block_size=8).generate(p, greedy, 14) for p in prompts]
    # 32 tokens of cache in all: each request needs a third page when both hold two
    engine = engine_for(folders["B"], dtype, block_size=8, num_blocks=4)
    ids = [engine.add_request(p, greedy, 14) for p in prompts]
    engine.run_until_done()
    assert engine.preemptions() > 0
    same_or_near_tie(folders["B"], prompts, [engine.output(i) for i in ids], alone, dtype)
    assert engine.runner.cache.free_pages() == [4]
    engine.runner.cache.check()


def test_temperature_sampling_does_not_depend_on_batching_or_preemption(folders):
    from from_scratch_inference_engine_b200 import SamplingParams
    params = [SamplingParams(temperature=0.8, seed=11),
              SamplingParams(temperature=1.3, top_k=20, top_p=0.9, seed=12),
              SamplingParams(temperature=0.0)]
    prompts = [helpers.random_ids(384, n, s) for n, s in ((7, 1), (30, 2), (12, 3))]
    alone = [engine_for(folders["B"], block_size=8).generate(p, q, 12)
             for p, q in zip(prompts, params)]
    assert len({tuple(o) for o in alone}) == 3
    together = engine_for(folders["B"], block_size=8)
    ids = [together.add_request(p, q, 12) for p, q in zip(prompts, params)]
    together.run_until_done()
    assert [together.output(i) for i in ids] == alone
    tight = engine_for(folders["B"], block_size=8, num_blocks=8)      # 64 tokens: forces preemption
    ids = [tight.add_request(p, q, 12) for p, q in zip(prompts, params)]
    tight.run_until_done()
    assert tight.preemptions() > 0 and [tight.output(i) for i in ids] == alone
    # another seed gives another continuation
    other = engine_for(folders["B"], block_size=8).generate(
        prompts[0], SamplingParams(temperature=0.8, seed=99), 12)
    assert other != alone[0]


def test_eos_stops_and_is_kept(folders):
    from from_scratch_inference_engine_b200 import SamplingParams
    greedy = SamplingParams(temperature=0.0)
    prompt = helpers.random_ids(256, 9, 8)
    free_run = engine_for(folders["A"]).generate(prompt, greedy, 10)
    eos = free_run[4]
    out = engine_for(folders["A"]).generate(prompt, greedy, 10, eos_id=eos)
    assert out == free_run[:free_run.index(eos) + 1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefix_cache_on_equals_off_with_hits(folders, dtype):
    from from_scratch_inference_engine_b200 import SamplingParams
    greedy = SamplingParams(temperature=0.0)
    shared = helpers.random_ids(384, 26, 9)
    tails = [helpers.random_ids(384, 5, s) for s in (1, 2, 3)]
    outs = {}
    for on in (False, True):
        engine = engine_for(folders["B"], dtype, block_size=8, enable_prefix_cache=on)
        outs[on] = [engine.generate(shared + tail, greedy, 6) for tail in tails]
        assert (engine.prefix_hits() > 0) == on
        engine.runner.cache.check()
    same_or_near_tie(folders["B"], [shared + t for t in tails], outs[True], outs[False], dtype)


def test_windowed_model_generates_within_a_small_window_pool(folders):
    """Config C: one full layer and two layers with a window of 21 keys.  The windowed
    group gets 6 pages of 8; a 100-token context passes through them."""
    from from_scratch_inference_engine_b200 import SamplingParams
    greedy = SamplingParams(temperature=0.0)
    prompt = helpers.random_ids(331, 70, 4)
    engine = engine_for(folders["C"], block_size=8, num_blocks=[16, 6])
    out = engine.generate(prompt, greedy, 30)
    assert assert_greedy_agrees(folders["C"], prompt, out, 1e-5) == 30
    assert engine.runner.cache.free_pages() == [16, 6]


def test_requests_beyond_the_pool_are_refused(folders):
    engine = engine_for(folders["A"], num_blocks=4)
    with pytest.raises(ValueError, match="page pool"):
        engine.add_request(list(range(10)), None, 8)
    with pytest.raises(IndexError):
        engine.add_request([1, 256], None, 2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_steps_give_the_same_tokens_as_one_step_at_a_time(folders, dtype):
    """The engine launches a step before it has read the tokens of the step before it (their
    ids enter the batch on the device).  Same outputs as without the overlap, with requests
    that stop at an end-of-sequence token (one token run for nothing and dropped), stop at
    their length, are preempted under a tight pool and share a prefix."""
    from from_scratch_inference_engine_b200 import SamplingParams
    shared = helpers.random_ids(384, 19, 77)
    prompts = [helpers.random_ids(384, n, s) for n, s in ((5, 1), (33, 2), (12, 3), (47, 4), (2, 5))]
    prompts += [shared + helpers.random_ids(384, 4, 6), shared + helpers.random_ids(384, 9, 7)]
    params = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.9, seed=5),
              SamplingParams(temperature=0.0), SamplingParams(temperature=1.2, top_k=30, seed=6),
              SamplingParams(temperature=0.0), SamplingParams(temperature=0.0),
              SamplingParams(temperature=0.7, top_p=0.8, seed=7)]
    if dtype == "bfloat16":
        # a draw near a step of the distribution would tell nothing about the overlap: greedy only
        params = [SamplingParams(temperature=0.0)] * len(params)
    lengths = [9, 14, 1, 11, 20, 7, 13]
    free_run = engine_for(folders["B"], dtype, block_size=8, pipeline=False).generate(prompts[4], params[4], 20)
    eos = {4: free_run[6]}                       # request 4 stops where that token first appears
    stopped = free_run[:free_run.index(free_run[6]) + 1]
    results = {}
    for pipeline in (False, True):
        for blocks in (64, 9):                   # roomy; 72 tokens of cache: forces preemption
            engine = engine_for(folders["B"], dtype, block_size=8, num_blocks=blocks, max_batch=4,
                                enable_prefix_cache=True, pipeline=pipeline)
            ids = [engine.add_request(p, q, n, eos_id=eos.get(i, -1))
                   for i, (p, q, n) in enumerate(zip(prompts, params, lengths))]
            engine.run_until_done()
            assert not engine.has_work()
            results[pipeline, blocks] = [list(engine.output(i)) for i in ids]
            engine.runner.cache.check()
            if blocks == 9:
                assert engine.preemptions() > 0
            engine.runner.raise_on_device_error()
    first = results[False, 64]
    if dtype == "float32":
        assert first[4] == stopped and len(stopped) < 20
        assert [len(o) for o in first] == [9, 14, 1, 11, len(stopped), 7, 13]
        assert all(other == first for other in results.values())
        return
    for outputs in results.values():
        for index, (prompt, out) in enumerate(zip(prompts, outputs)):
            if index == 4:        # stops at its end-of-sequence token, wherever that comes
                assert out[-1] == eos[4] or len(out) == 20
                assert eos[4] not in out[:-1]
            else:
                assert len(out) == lengths[index]
            assert_greedy_agrees(folders["B"], prompt, out, 2e-2)


def test_warm_up_captures_the_decode_graphs_and_changes_no_token(folders):
    from from_scratch_inference_engine_b200 import SamplingParams
    greedy = SamplingParams(temperature=0.0)
    prompts = [helpers.random_ids(384, n, s) for n, s in ((9, 1), (20, 2), (3, 3))]
    cold = engine_for(folders["B"], block_size=8, dtype="bfloat16")
    want = [cold.generate(p, greedy, 8) for p in prompts]
    warm = engine_for(folders["B"], block_size=8, dtype="bfloat16", max_batch=4)
    graphs = warm.warm_up(100)
    assert graphs == 3 and len(warm.runner._graphs) == 3          # batches 1, 2 and 4 at one table width
    ids = [warm.add_request(p, greedy, 8) for p in prompts]
    warm.run_until_done()
    assert len(warm.runner._graphs) == 3                            # nothing was captured while serving
    assert sorted(warm.output(i) for i in ids) == sorted(want)


def test_command_line_generates_from_a_random_weights_folder(tmp_path, capsys):
    """The command line writes a random model from a configuration, generates for several requests
    and reports JSON; the same tokens as the Python entry point on that folder."""
    import json
    from from_scratch_inference_engine_b200 import LLM, GenerationConfig, cli
    config = dict(helpers.TINY["E"]["config"])
    config_path = tmp_path / "config_in.json"
    config_path.write_text(json.dumps(config))
    folder = tmp_path / "model"
    code = cli.main(["--model-dir", str(folder), "--random-weights", str(config_path), "--weights-seed", "5",
                     "--std", "0.08", "--prompt-ids", "5,17,3,88,41", "--num-requests", "3", "--max-tokens", "9",
                     "--block-size", "16", "--num-blocks", "32", "--json"])
    assert code == 0
    report = json.loads(capsys.readouterr().out)
    assert report["requests"] == 3 and report["total_output_tokens"] == 27
    assert report["outputs"][0] == report["outputs"][1] == report["outputs"][2]      # greedy, same prompt
    assert (folder / "config.json").exists() and (folder / "model.safetensors").exists()
    llm = LLM(str(folder), block_size=16, num_blocks=32)
    assert llm.generate_ids([5, 17, 3, 88, 41], GenerationConfig(max_tokens=9, temperature=0.0)) == report["outputs"][0]


@pytest.mark.parametrize("pipeline", [False, True])
def test_engine_raises_when_a_kernel_has_set_the_error_flag(folders, pipeline):
    """Kernels that refuse an input or give up a wait set a flag on the device; it travels to the
    host with the sampled ids, and the engine raises instead of handing out tokens.  (The flag is
    set by hand here: nothing is made to fail on the GPU.)"""
    from from_scratch_inference_engine_b200 import SamplingParams
    from from_scratch_inference_engine_b200.engine.runner import DeviceFault
    engine = engine_for(folders["A"], block_size=4, num_blocks=32, max_batch=2, pipeline=pipeline)
    engine.add_request(helpers.random_ids(256, 9, 1), SamplingParams(temperature=0.0), 6)
    assert engine.step() > 0
    engine.runner.error.fill_(12)
    with pytest.raises(DeviceFault, match="tile never arrived"):
        engine.run_until_done()
