"""The engine against the plain implementation at the Qwen2.5-7B layer sizes.

Hidden 3,584, 28 query heads over 4 kv heads of 128, intermediate 18,944, vocabulary 152,064,
untied head, theta 1e6 - with 2 of the shape's 28 layers, so that the float32 weights (6 GB) and
the float64 plain run fit beside everything else a test run holds; set FSIE_SHAPE_LAYERS=28 for
all of them (about 100 GB of GPU memory and a few minutes).  Random bf16 weights N(0, 0.02) are
drawn once on the GPU and given both to the engine and to the plain implementation
(tests/plain_qwen2.py, float64, on the GPU, one tensor widened at a time).  Four requests are
replayed whole, with the last 32 tokens one by one, in portions of changing size, mixed, and
mixed with a release in the middle and a second run from position 0 - through a page pool that
holds just what the live requests need - in float32, in bfloat16 as the engine chooses its
kernels, and in bfloat16 with the tiled tcgen05 product and the tcgen05 attention for decoded
tokens forced onto these few tokens.
"""

import os

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

LAYERS = int(os.environ.get("FSIE_SHAPE_LAYERS", "2"))
SHAPE = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=LAYERS,
             hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
             intermediate_size=18944, vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6,
             tie_word_embeddings=False, max_position_embeddings=32768, use_sliding_window=False)
LENGTHS = {"a": 150, "b": 72, "c": 48, "d": 33}
# relative to max(1, largest |plain logit| of the row).  float32: the reference's own bar between
# its modes (tests/cpp/test_cuda_model.cpp:57, 66); 7.9e-6 was seen.  bfloat16: 2.5 times what was
# seen on a B200 (the terminal summary prints it): 1.8e-2 at 2 layers against the exact plain
# logits, 1.2e-2 against the plain implementation that stores every result in bfloat16 as the
# engine does; rounding accumulates with depth: 28 layers were seen at 7.3e-2 and 4.8e-2 (float32: 3.3e-5).
BOUND = {"float32": 1e-4, "bfloat16": 4.4e-2 if LAYERS <= 2 else 1.8e-1}
BOUND_STORED = 3.0e-2 if LAYERS <= 2 else 1.2e-1
PAGE = 16


@pytest.fixture(scope="module")
def shape_model():
    """(configuration, tensors on the GPU, requests, plain float64 logits per request)."""
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.parts import tensor_specs
    from from_scratch_inference_engine_b200.weights.random_init import random_tensors_on_device
    config = config_from_dict(dict(SHAPE))
    tensors = random_tensors_on_device(tensor_specs(config.build_spec()), seed=0, std=0.02,
                                       device="cuda")
    requests = {key: helpers.random_ids(config.vocab_size, n, seed)
                for seed, (key, n) in enumerate(LENGTHS.items())}

    class Widening(dict):                      # one tensor in float64 at a time
        def __getitem__(self, name):
            return tensors[name].double()

        def __contains__(self, name):
            return name in tensors
    plain_config = plain.read_config_dict(dict(SHAPE))
    want = {key: plain.forward(plain_config, Widening(), ids).cpu().numpy()
            for key, ids in requests.items()}
    plain_config["store"] = torch.bfloat16
    stored = {key: plain.forward(plain_config, Widening(), ids).cpu().numpy()
              for key, ids in requests.items()}
    yield config, tensors, requests, want, stored
    tensors.clear()
    torch.cuda.empty_cache()


FAMILIES = {
    "whole": lambda r: (helpers.trace_whole(r), r),
    "tail": lambda r: (helpers.trace_tail_by_one(r), r),
    "portions": lambda r: (helpers.trace_portions(r, 5), r),
    "mixed": lambda r: (helpers.trace_mixed(r, 5), r),
    "recompute": lambda r: helpers.trace_mixed_with_recompute(r, 5),
}
MODES = {
    "float32": ("float32", {}),
    "bfloat16": ("bfloat16", {}),
    # every product of more than 16 tokens through the tiled tcgen05 kernel, decoded tokens and
    # short portions through the tcgen05 attention kernel, however few tiles and blocks that makes
    "bfloat16-tcgen05-forced": ("bfloat16", {"tiled_min_tiles": 1, "decode_tcgen05_min_blocks": 1}),
}


@pytest.mark.parametrize("mode", list(MODES))
def test_replay_at_the_7b_layer_sizes(shape_model, mode):
    from from_scratch_inference_engine_b200.engine import LoadedModel, ModelRunner
    from from_scratch_inference_engine_b200.kernels import ops
    config, tensors, requests, want, stored = shape_model
    dtype, options = MODES[mode]
    model = LoadedModel.from_tensors(config, tensors, dtype=dtype, max_positions=512, **options)
    calls = {"gemm_tiles": 0, "attention_tc_decode": 0}
    originals = {name: getattr(ops, name) for name in calls}

    def counting(name):
        def call(*args, **kwargs):
            calls[name] += 1
            return originals[name](*args, **kwargs)
        return call
    for name in calls:
        setattr(ops, name, counting(name))
    try:
        report = {}
        for family, make in FAMILIES.items():
            steps, names = make(requests)
            need = helpers.live_tokens_needed(steps, round_to=PAGE)
            runner = ModelRunner(model.model, model.runtime, page_size=PAGE, num_pages=need // PAGE,
                                 max_requests=4)
            rows = helpers.run_trace_in_process(runner, steps)
            assert len(rows) == sum(len(e["tokens"]) for s in steps for e in s["entries"])
            worst, worst_stored, bad, disagree = 0.0, 0.0, [], 0
            for (key, pos), row in rows.items():
                target = want[key.split("~")[0]][pos]
                base = max(1.0, float(np.abs(target).max()))
                diff = float(np.abs(row - target).max()) / base
                worst = max(worst, diff)
                if diff > BOUND[dtype]:
                    bad.append((key, pos, diff))
                disagree += int(row.argmax()) != int(target.argmax())
                if dtype == "bfloat16":
                    diff = float(np.abs(row - stored[key.split("~")[0]][pos]).max()) / base
                    worst_stored = max(worst_stored, diff)
                    if diff > BOUND_STORED:
                        bad.append((key, pos, diff, "against plain stored in bfloat16"))
            report[family] = worst
            helpers.OBSERVED[f"7B sizes, {LAYERS} layers, {mode}, {family}"] = worst
            if dtype == "bfloat16":
                helpers.OBSERVED[f"7B sizes, {LAYERS} layers, {mode}, {family}, against plain "
                                 f"stored in bfloat16"] = worst_stored
            assert not bad, f"{family}: {len(bad)} rows beyond their bound, first {bad[:3]}"
            if dtype == "float32":
                assert disagree == 0, f"{family}: argmax differs at {disagree} positions"
            assert all(pool.num_free == pool.num_pages for pool in runner.cache.pools)
            del runner
    finally:
        for name, original in originals.items():
            setattr(ops, name, original)
    if mode == "bfloat16-tcgen05-forced":
        assert calls["gemm_tiles"] > 0 and calls["attention_tc_decode"] > 0
    if dtype == "float32":
        # Cutting the work differently moves nothing beyond rounding.  Steps of up to 48 tokens and
        # longer ones take float32 product kernels that add in different orders (a tree over 32
        # lanes; one chain over k): at 2 layers every family showed the same 7.9e-6, at 28 layers
        # the families of long steps 3.3e-5 and those of short steps 7.8e-6.
        assert max(report.values()) - min(report.values()) < 5e-5
