"""The engine against the plain implementation under every way of cutting the work."""

import numpy as np
import pytest
import torch

import helpers
from helpers import TINY

pytestmark = pytest.mark.gpu

# float32: the engine's 32-bit sums against the plain 64-bit ones.  bfloat16: every operation's
# result is stored with 8 bits of mantissa, and how far that moves the logits depends on the
# model (depth, widths, size of the weights), so each configuration has its own bound: 2.5 times
# the largest difference seen over all families and kernel choices on a B200 (the terminal
# summary of a GPU run prints what it saw: A 2.5e-3, B 1.5e-2, C 1.2e-2, D 1.5e-2, E 1.5e-2,
# F 8.8e-3).  All bounds are relative to max(1, the row's largest |logit|).
# The bfloat16 engine is also compared with the plain implementation that stores results in
# bfloat16 where the engine does (plain_qwen2.stored_as, and the attention weights).  On a
# whole sequence of config A the two then agree to 2e-7: the model of the rounding points is
# right.  It does not give a sharper bound in general: once a context spans more than one
# tile of keys the engine rounds its attention weights against a running maximum, values
# differ by a fraction of a bfloat16 step, every later rounding falls independently, and the
# difference is as large as against the exact logits.  The same bound holds for both.
FLOAT32_BOUND = 1e-4
BFLOAT16_BOUND = {"A": 6.4e-3, "B": 3.8e-2, "C": 3.0e-2, "D": 3.9e-2, "E": 3.9e-2, "F": 2.2e-2}


def assert_rows_match_plain(rows, requests, folder, dtype, name):
    if dtype == "float32":
        worst, scale, bad = helpers.compare_rows(rows, requests, folder, FLOAT32_BOUND,
                                                 f"float32 {name}")
    else:
        worst, scale, bad = helpers.compare_rows(rows, requests, folder, BFLOAT16_BOUND[name],
                                                 f"bfloat16 {name} against exact plain")
        assert not bad, f"{len(bad)} rows differ, first {bad[:3]}, worst {worst:.3e} at scale {scale:.3f}"
        worst, scale, bad = helpers.compare_rows(rows, requests, folder, BFLOAT16_BOUND[name],
                                                 f"bfloat16 {name} against plain stored in bfloat16",
                                                 store=torch.bfloat16)
    assert not bad, f"{len(bad)} rows differ, first {bad[:3]}, worst {worst:.3e} at scale {scale:.3f}"


REQUESTS = {
    "A": {"a": 100, "b": 37, "c": 64, "d": 81, "e": 5, "f": 49},
    "B": {"a": 130, "b": 33, "c": 100, "d": 64, "e": 7, "f": 1 + 32},
    "C": {"a": 150, "b": 40, "c": 97, "d": 64, "e": 23},
    "D": {"a": 70, "b": 35, "c": 48},
    "E": {"a": 300, "b": 150, "c": 90, "d": 64},
    "F": {"a": 290, "b": 150, "c": 129, "d": 64},
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model_dir(root, name) for name in TINY}


def requests_for(name):
    vocab = TINY[name]["config"]["vocab_size"]
    return {key: helpers.random_ids(vocab, n, seed=sum(map(ord, name + key)))
            for key, n in REQUESTS[name].items()}


def build_runner(folder, dtype, max_tokens, page_size, **runtime_options):
    from from_scratch_inference_engine_b200.engine import LoadedModel, ModelRunner
    pages = -(-max_tokens // page_size)
    model = LoadedModel.from_pretrained(folder, dtype=dtype, max_positions=pages * page_size,
                                        **runtime_options)
    return ModelRunner(model.model, model.runtime, page_size=page_size, num_pages=pages,
                       max_requests=8)


FAMILIES = {
    "whole": lambda r, seed: (helpers.trace_whole(r), r),
    "tail": lambda r, seed: (helpers.trace_tail_by_one(r), r),
    "portions": lambda r, seed: (helpers.trace_portions(r, seed), r),
    "mixed": lambda r, seed: (helpers.trace_mixed(r, seed), r),
    # released in the middle and fed again from position 0 (preemption with recompute)
    "recompute": helpers.trace_mixed_with_recompute,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("name,page_size", [("A", 4), ("B", 8), ("C", 16), ("D", 16), ("E", 16),
                                            ("F", 32)])
def test_replay_matches_plain(folders, name, page_size, family, dtype):
    steps, requests = FAMILIES[family](requests_for(name), 11)
    # the pool holds exactly what the live requests need, so pages are used again
    need = helpers.live_tokens_needed(steps, round_to=page_size)
    runner = build_runner(folders[name], dtype, need, page_size)
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) == sum(len(e["tokens"]) for step in steps for e in step["entries"])
    if family != "recompute":
        assert len(rows) == sum(len(v) for v in requests.values())
    assert_rows_match_plain(rows, requests, folders[name], dtype, name)
    assert all(pool.num_free == pool.num_pages for pool in runner.cache.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
    """Positions 0, 1, 2 alone: one key, no history, the first page."""
    requests = {"x": helpers.random_ids(256, 3, 5)}
    for steps in (helpers.trace_whole(requests), helpers.trace_tail_by_one(requests, tail=2)):
        runner = build_runner(folders["A"], dtype, 64, 4)
        rows = helpers.run_trace_in_process(runner, steps)
        assert_rows_match_plain(rows, requests, folders["A"], dtype, "A")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """A short prompt, then 200 tokens one by one across many pages."""
    ids = helpers.random_ids(384, 230, 9)
    requests = {"x": ids}
    steps = helpers.trace_tail_by_one(requests, tail=200)
    runner = build_runner(folders["B"], dtype, 256, 8)
    rows = helpers.run_trace_in_process(runner, steps)
    assert_rows_match_plain(rows, requests, folders["B"], dtype, "B")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps_equal_uncaptured_ones(folders, dtype):
    """Steps of single tokens replay CUDA graphs; the same kernels launched one by one give
    the same logits beyond rounding (a graph is captured for a rounded-up table width and
    may split the keys otherwise), across batch sizes that change and tables that grow."""
    requests = requests_for("B")
    steps = helpers.trace_mixed(requests, seed=7, decode_tail=20)
    need = helpers.live_tokens_needed(steps, round_to=8)
    runner = build_runner(folders["B"], dtype, need, 8)
    assert runner.cuda_graphs
    captured = helpers.run_trace_in_process(runner, steps)
    assert runner._graphs, "no decode step went through a graph"
    plain_runner = build_runner(folders["B"], dtype, need, 8)
    plain_runner.cuda_graphs = False
    direct = helpers.run_trace_in_process(plain_runner, steps)
    assert captured.keys() == direct.keys()
    if dtype == "float32":
        for key, row in captured.items():
            assert np.abs(row - direct[key]).max() < 2e-5, key
    for rows in (captured, direct):
        assert_rows_match_plain(rows, requests, folders["B"], dtype, "B")


def test_cutting_does_not_change_float32_beyond_rounding(folders):
    """The same request whole and in portions: rows agree far inside the tolerance."""
    requests = {"x": helpers.random_ids(384, 90, 3)}
    results = []
    for steps in (helpers.trace_whole(requests), helpers.trace_portions(requests, 4),
                  helpers.trace_tail_by_one(requests)):
        runner = build_runner(folders["B"], "float32", 128, 8)
        results.append(helpers.run_trace_in_process(runner, steps))
    for other in results[1:]:
        for key, row in results[0].items():
            assert np.abs(row - other[key]).max() < 2e-5


@pytest.mark.parametrize("family", ["tail", "mixed"])
@pytest.mark.parametrize("name,page_size", [("B", 8), ("C", 16), ("D", 16)])
def test_replay_with_the_few_token_product_on_every_matrix(folders, name, page_size, family):
    """The tcgen05 product that steps of up to 16 tokens use is reserved for large matrices;
    here it is forced onto the tiny models' matrices so that replay covers it too."""
    steps, requests = FAMILIES[family](requests_for(name), 11)
    need = helpers.live_tokens_needed(steps, round_to=page_size)
    runner = build_runner(folders[name], "bfloat16", need, page_size, few_token_min_elements=0)
    assert runner.runtime._few_token_weights
    rows = helpers.run_trace_in_process(runner, steps)
    assert_rows_match_plain(rows, requests, folders[name], "bfloat16", name)


@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
@pytest.mark.parametrize("name,page_size", [("B", 8), ("C", 16), ("E", 16)])
def test_replay_with_the_tiled_product_on_every_matrix(folders, name, page_size, family, monkeypatch):
    """Steps of more than 16 tokens take the tiled tcgen05 product (bias and SwiGLU in its
    epilogue) for every matrix, however few tiles that makes at these sizes."""
    steps, requests = FAMILIES[family](requests_for(name), 5)
    need = helpers.live_tokens_needed(steps, round_to=page_size)
    runner = build_runner(folders[name], "bfloat16", need, page_size, tiled_min_tiles=1)
    assert runner.runtime._tiled_weights
    from from_scratch_inference_engine_b200.kernels import ops
    calls, original = [], ops.gemm_tiles
    monkeypatch.setattr(ops, "gemm_tiles", lambda *a, **k: (calls.append(1), original(*a, **k))[1])
    rows = helpers.run_trace_in_process(runner, steps)
    assert_rows_match_plain(rows, requests, folders[name], "bfloat16", name)
    assert len(calls) >= 4 * len(runner.model.blocks)


@pytest.mark.parametrize("family", ["tail", "portions", "mixed"])
def test_replay_with_the_tcgen05_kernel_for_decoded_tokens(folders, family, monkeypatch):
    """Decoded tokens and portions of up to 16 rows take the tcgen05 attention kernel only when
    they fill the GPU; here it is forced onto a handful of requests (head size 128)."""
    steps, requests = FAMILIES[family](requests_for("F"), 7)
    need = helpers.live_tokens_needed(steps, round_to=16)
    runner = build_runner(folders["F"], "bfloat16", need, 16, decode_tcgen05_min_blocks=1)
    from from_scratch_inference_engine_b200.kernels import ops
    calls, original = [], ops.attention_tc_decode
    monkeypatch.setattr(ops, "attention_tc_decode",
                        lambda *a, **k: (calls.append(1), original(*a, **k))[1])
    rows = helpers.run_trace_in_process(runner, steps)
    assert_rows_match_plain(rows, requests, folders["F"], "bfloat16", "F")
    assert calls
    if family == "tail":
        assert runner._graphs, "the decoded tokens did not go through a captured step"


ODD = {
    # nothing a multiple of anything: head size 20 (no tensor-core attention, the 32-bit kernel on
    # bfloat16 storage), widths that are no multiples of 8 (no 16-byte rows for the own products)
    "all odd": dict(hidden_size=100, num_attention_heads=5, num_key_value_heads=5, head_dim=20,
                    intermediate_size=37, vocab_size=101, tie_word_embeddings=False),
    # 33 heads in groups of 3, head size 16, a prime vocabulary, tied head
    "many small heads": dict(hidden_size=264, num_attention_heads=33, num_key_value_heads=11,
                             head_dim=16, intermediate_size=1000, vocab_size=4099,
                             tie_word_embeddings=True),
    # head size 112 (a multiple of 16 that is neither 64 nor 128), pages of 5 tokens
    "head 112": dict(hidden_size=256, num_attention_heads=2, num_key_value_heads=2, head_dim=112,
                     intermediate_size=520, vocab_size=777, tie_word_embeddings=False),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("all odd", 16), ("many small heads", 8), ("head 112", 5)])
def test_replay_at_sizes_that_fit_no_tile(tmp_path, name, page_size, dtype):
    """Sizes that the fast kernels do not take must fall to kernels that do, never to a wrong
    result: mixed steps with a release and a second run, against the plain implementation.
    (bfloat16 bound: 2.5 times what these three were seen at, 3.3e-2 at most.)"""
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.weights import write_random_model
    config = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2,
                  rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=512, **ODD[name])
    folder = write_random_model(tmp_path / "odd", config_from_dict(config), 3, 0.1, torch.bfloat16)
    requests = {k: helpers.random_ids(config["vocab_size"], n, i)
                for i, (k, n) in enumerate({"a": 150, "b": 40, "c": 97, "d": 3}.items())}
    steps, names = helpers.trace_mixed_with_recompute(requests, 3)
    need = helpers.live_tokens_needed(steps, round_to=page_size)
    runner = build_runner(folder, dtype, need, page_size)
    rows = helpers.run_trace_in_process(runner, steps)
    worst, scale, bad = helpers.compare_rows(rows, names, folder, 1e-4 if dtype == "float32" else 8e-2,
                                             f"{dtype} {name}")
    assert not bad, f"{len(bad)} rows differ, first {bad[:3]}, worst {worst:.3e} at scale {scale:.3f}"
    assert all(pool.num_free == pool.num_pages for pool in runner.cache.pools)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,page_size", [(26, 32), (61, 16), (200, 16)])
def test_replay_window_that_starts_inside_a_tile_of_keys(tmp_path, window, page_size, dtype):
    """Windowed layers at a head size the tcgen05 attention takes, prompts long enough that a
    portion's key range is cut in two: the window of a token just behind a tile's edge reaches
    back into the tile before it, which one range must see and no range twice.
    (One layer: its bfloat16 results were seen at 1.4e-2 to 2.4e-2 of the row's largest logit, the
    bound is 2.5 times that; a key counted twice moved them by 1.6e-1 to 2.2e-1.)"""
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.weights import write_random_model
    config = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=1,
                  rope_theta=1e6, rms_norm_eps=1e-5, max_position_embeddings=1024, hidden_size=300,
                  num_attention_heads=16, num_key_value_heads=4, head_dim=128, intermediate_size=356,
                  vocab_size=1575, tie_word_embeddings=True, use_sliding_window=True,
                  sliding_window=window, max_window_layers=0)
    folder = write_random_model(tmp_path / "window", config_from_dict(config), 21, 0.1, torch.bfloat16)
    requests = {k: helpers.random_ids(config["vocab_size"], n, i)
                for i, (k, n) in enumerate({"a": 238, "b": 106, "c": 307, "d": 72}.items())}
    for family, (steps, names) in (("tail", (helpers.trace_tail_by_one(requests, 20), requests)),
                                   ("recompute", helpers.trace_mixed_with_recompute(requests, 21))):
        need = helpers.live_tokens_needed(steps, round_to=page_size)
        runner = build_runner(folder, dtype, need, page_size)
        rows = helpers.run_trace_in_process(runner, steps)
        worst, scale, bad = helpers.compare_rows(rows, names, folder, 1e-4 if dtype == "float32" else 6e-2,
                                                 f"{dtype} window {window} {family}")
        assert not bad, f"{family}: {len(bad)} rows differ, first {bad[:3]}, worst {worst:.3e} at scale {scale:.3f}"
