"""Each part alone, built from a PartSpec with its own sizes, against the plain functions;
then run orders that name a layer twice or let a layer read another layer's cache."""

import dataclasses
import math

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain
from helpers import TINY, OnePartModel

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def tol(dtype):
    return 3e-5 if dtype == "float32" else 3e-2


def runtime_for(dtype, max_positions=4096):
    from from_scratch_inference_engine_b200.engine import Runtime
    return Runtime("cuda:0", dtype, max_positions=max_positions)


def bound_part(role, spec, prefix, runtime, seed=0, std=0.3):
    """Build a part from its spec, draw its tensors, bind them; returns (part, float64 tensors)."""
    from from_scratch_inference_engine_b200.parts import build_part
    from from_scratch_inference_engine_b200.weights import random_tensors, to_runtime_dtype
    part = build_part(role, spec, prefix)
    specs = part.tensor_specs()
    drawn = random_tensors(specs, seed, std, torch.bfloat16)
    by_name = {s.name: s for s in specs}
    part.bind({n: to_runtime_dtype(t, by_name[n], runtime.dtype).to(runtime.device)
               for n, t in drawn.items()}, runtime)
    return part, {n: t.double() for n, t in drawn.items()}


def close(got, want, dtype):
    got = got.detach().double().cpu()
    assert got.shape == want.shape
    err = (got - want).abs().max().item()
    assert err < tol(dtype) * max(1.0, want.abs().max().item()), f"error {err:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from from_scratch_inference_engine_b200.config import PartSpec
    rt = runtime_for(dtype)
    norm, w = bound_part("norm", PartSpec("rmsnorm", {"width": 200, "eps": 1e-3}), "n.", rt)
    assert [s.name for s in norm.tensor_specs()] == ["n.weight"]
    x0 = torch.randn(5, 200, generator=torch.Generator().manual_seed(0))
    delta = torch.randn(5, 200, generator=torch.Generator().manual_seed(1)).to(rt.dtype)
    x = x0.cuda()
    y = norm.forward(x, delta.cuda())
    close(y, plain.rms_norm(x0.double() + delta.double(), w["n.weight"], 1e-3), dtype)
    close(x, x0.double() + delta.double(), "float32")


def test_rotary_table_matches_the_reference_formula():
    from from_scratch_inference_engine_b200.parts.rope import rotary_table
    table = rotary_table(1e6, 64, 5000)
    for pos in (0, 1, 777, 4999):
        for i in (0, 5, 31):
            ang = pos * (1e6 ** (-2.0 * i / 64))
            assert table[pos, i] == np.float32(math.cos(ang))
            assert table[pos, 32 + i] == np.float32(math.sin(ang))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from from_scratch_inference_engine_b200.config import PartSpec
    rt = runtime_for(dtype)
    mlp, w = bound_part("feed_forward", PartSpec("swiglu", {"hidden_size": 72,
                                                            "intermediate_size": 200}), "m.", rt)
    y0 = torch.randn(11, 72, generator=torch.Generator().manual_seed(2)).to(rt.dtype)
    got = mlp.forward(None, y0.cuda())
    y = y0.double()
    want = plain.linear(plain.silu_mul(plain.linear(y, w["m.gate_proj.weight"]),
                                       plain.linear(y, w["m.up_proj.weight"])),
                        w["m.down_proj.weight"])
    close(got, want, dtype)


def attention_spec(position, window=0, bias=True):
    from from_scratch_inference_engine_b200.config import PartSpec
    return PartSpec("gqa_attention", {"hidden_size": 80, "num_heads": 6, "num_kv_heads": 3,
                                      "head_dim": 32, "qkv_bias": bias, "window": window,
                                      "position": position})


def plain_attention_part(w, y, theta, window, bias, rotary=True):
    def project(name):
        b = w[f"a.{name}_proj.bias"] if bias else None
        return plain.linear(y, w[f"a.{name}_proj.weight"], b)
    q, k, v = project("q"), project("k"), project("v")
    positions = list(range(y.shape[0]))
    if rotary:
        q, k = plain.rope(q, 6, 32, theta, positions), plain.rope(k, 3, 32, theta, positions)
    return plain.linear(plain.attention(q, k, v, 6, 3, 32, 0, window), w["a.o_proj.weight"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("variant", ["rotary", "no_position", "window", "no_bias"])
def test_attention_part_through_the_cache(dtype, variant):
    """The mixer alone: two requests, fed in portions, through real pages."""
    from from_scratch_inference_engine_b200.config import PartSpec
    from from_scratch_inference_engine_b200.engine import ModelRunner, StepEntry
    rt = runtime_for(dtype)
    position = PartSpec("none") if variant == "no_position" else \
        PartSpec("rotary", {"theta": 3e4, "rotary_dim": 32, "max_position": 0})
    window = 9 if variant == "window" else 0
    bias = variant != "no_bias"
    mixer, w = bound_part("mixer", attention_spec(position, window, bias), "a.", rt)
    assert mixer.cache_need().window == window
    model = OnePartModel(mixer, lambda ctx, y, cache: mixer.forward(ctx, y, cache))
    runner = ModelRunner(model, rt, page_size=4, num_pages=24, max_requests=4)
    gen = torch.Generator().manual_seed(3)
    inputs = {"a": torch.randn(31, 80, generator=gen).to(rt.dtype),
              "b": torch.randn(18, 80, generator=gen).to(rt.dtype)}
    handles = {k: runner.cache.open(k) for k in inputs}
    got = {k: [] for k in inputs}
    # portions: a 13 | a 1 + b 18 | a 17 (one batch holds a decode token beside a prompt)
    for batch in ([("a", 13)], [("a", 1), ("b", 18)], [("a", 17)]):
        model.inputs = torch.cat([inputs[k][len(torch.cat(got[k])) if got[k] else 0:][:n]
                                  for k, n in batch]).cuda()
        runner.step([StepEntry(handles[k], [0] * n) for k, n in batch])
        at = 0
        for k, n in batch:
            got[k].append(model.outputs[at:at + n].cpu())
            at += n
    for k in inputs:
        want = plain_attention_part(w, inputs[k].double(), 3e4, window, bias,
                                    rotary=variant != "no_position")
        close(torch.cat(got[k]), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_alone(dtype):
    from from_scratch_inference_engine_b200.config import config_from_dict
    from from_scratch_inference_engine_b200.engine import ModelRunner, StepEntry
    from from_scratch_inference_engine_b200.config import PartSpec
    rt = runtime_for(dtype)
    config = config_from_dict(TINY["D"]["config"])
    layer = config.build_spec().layers[1]
    block, w = bound_part("arrangement", PartSpec("prenorm", {"layer": layer}), layer.prefix, rt,
                          std=0.1)
    x0 = torch.randn(12, 96, generator=torch.Generator().manual_seed(5))
    delta = (0.1 * torch.randn(12, 96, generator=torch.Generator().manual_seed(6))).to(rt.dtype)
    state = {}

    def run(ctx, inputs, cache):
        x = x0.clone().cuda()
        state["delta"] = block.forward(ctx, x, delta.cuda(), cache)
        return x
    model = OnePartModel(block.mixer, run)
    runner = ModelRunner(model, rt, page_size=16, num_pages=2, max_requests=1)
    runner.step([StepEntry(runner.cache.open("x"), [0] * 12)])
    c = plain.read_config_dict(TINY["D"]["config"])
    weights = {k: v for k, v in w.items()}
    want, _ = plain.decoder_layer(c, weights, 1, x0.double() + delta.double(), list(range(12)))
    close(model.outputs.double().cpu() + state["delta"].double().cpu(), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("order", ["twice", "shared_cache"])
def test_run_order_is_data(tmp_path, dtype, order):
    """A layer named twice runs twice with the same weights and a cache entry per call; a
    call with writes_cache=False attends over the keys another call stored."""
    from from_scratch_inference_engine_b200.config import LayerCall, config_from_dict
    from from_scratch_inference_engine_b200.engine import ModelRunner, Runtime, StepEntry
    from from_scratch_inference_engine_b200.parts import DecoderModel
    from from_scratch_inference_engine_b200.weights import load_checkpoint
    folder = helpers.make_model_dir(tmp_path, "D")
    spec = config_from_dict(TINY["D"]["config"]).build_spec()
    calls = {"twice": (LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1)),
             "shared_cache": (LayerCall(0), LayerCall(1, cache=0, writes_cache=False),
                              LayerCall(1), LayerCall(0, cache=2, writes_cache=False))}[order]
    spec = dataclasses.replace(spec, schedule=calls)
    rt = runtime_for(dtype)
    model = DecoderModel(spec)
    model.bind(load_checkpoint(folder), rt)
    assert len(model.cache_needs()) == 4
    assert sum(n is not None for n in model.cache_needs()) == (4 if order == "twice" else 2)
    runner = ModelRunner(model, rt, page_size=8, num_pages=12, max_requests=2)
    ids = helpers.random_ids(200, 45, 1)
    handle = runner.cache.open("x")
    rows = []
    for lo, hi in ((0, 20), (20, 22), (22, 44), (44, 45)):
        logits = runner.step([StepEntry(handle, ids[lo:hi], list(range(hi - lo)))])
        rows.append(logits.cpu())
    config, weights = plain.load(folder)
    want = plain.forward(config, weights, ids, schedule=spec.resolved_schedule())
    close(torch.cat(rows), want, dtype)
    usual = plain.forward(config, weights, ids)
    assert (usual - want).abs().max().item() > 1e-3          # the order matters


@pytest.mark.parametrize("rows", [5, 40])
@pytest.mark.parametrize("route", ["own kernels", "float32 slabs"])
def test_logits_stay_32_bit_without_the_library_float32_result(rows, route):
    """Where torch cannot return a float32 product of bfloat16 operands, the output head must
    not round its logits to bfloat16 on the way (8 bits of mantissa: ~4e-3 relative)."""
    runtime = runtime_for("bfloat16")
    runtime._f32_out = False
    if route == "float32 slabs":
        runtime.products = "library"                  # none of the engine's products takes it
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, 72, generator=g).to(torch.bfloat16)
    w = torch.randn(333, 72, generator=g).to(torch.bfloat16)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        got = runtime.linear_f32_out(x.cuda(), w.cuda().contiguous())
    assert got.dtype is torch.float32 and got.shape == (rows, 333)
    want = x.double() @ w.double().t()
    assert (got.double().cpu() - want).abs().max().item() < 2e-5 * want.abs().max().item()
