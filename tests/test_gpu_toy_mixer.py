"""A mixer with state of its own, defined here, is registered, built and stepped without
any change to the package: the part registry, the architecture registry, the random
weights mode, the loader, the state slots, the step function and the scheduler carry it."""

import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu


HYBRID_HEADS, HYBRID_THETA = 2, 10000.0


def define_toy():
    from from_scratch_inference_engine_b200.config import (LayerCall, LayerSpec, ModelSpec,
                                                            PartSpec, register_architecture)
    from from_scratch_inference_engine_b200.parts import Mixer, StateNeed, register_part
    from from_scratch_inference_engine_b200.weights import TensorSpec

    @register_part("mixer", "toy_decaying_sum")
    class DecayingSum(Mixer):
        """s_t = decay * s_{t-1} + y_t per request; out_t = s_t W^T.  The state s is a vector
        of `width` floats per request that lives in a state slot, not in pages."""

        def __init__(self, prefix, width, decay):
            self.prefix, self.width, self.decay = prefix, width, decay

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "out.weight", (self.width, self.width))]

        def state_need(self):
            return StateNeed((self.width,), torch.float32)

        def bind(self, tensors, runtime):
            self.runtime = runtime
            self.weight = tensors[self.prefix + "out.weight"]

        def forward(self, ctx, y, cache):
            out = torch.empty_like(y, dtype=torch.float32)
            for i in range(ctx.num_items):
                start, count = int(ctx.h_qstart[i]), int(ctx.h_qlen[i])
                state = cache.state[int(ctx.h_slots[i])]
                for t in range(start, start + count):
                    state.mul_(self.decay).add_(y[t].float())
                    out[t] = state
            return self.runtime.linear(out.to(y.dtype), self.weight, None)

    @dataclass(frozen=True)
    class ToyConfig:
        width: int
        layers: int
        vocab: int
        decay: float
        eps: float
        attention_layers: int = 0      # this many leading layers mix by attention instead

        @classmethod
        def from_dict(cls, d):
            return cls(d["width"], d["layers"], d["vocab"], d["decay"], d["eps"],
                       d.get("attention_layers", 0))

        def to_dict(self):
            return {"architectures": ["ToyStateForCausalLM"], "width": self.width,
                    "layers": self.layers, "vocab": self.vocab, "decay": self.decay,
                    "eps": self.eps, "attention_layers": self.attention_layers}

        def build_spec(self):
            norm = PartSpec("rmsnorm", {"width": self.width, "eps": self.eps})
            attention = PartSpec("gqa_attention", {
                "hidden_size": self.width, "num_heads": HYBRID_HEADS, "num_kv_heads": 1,
                "head_dim": self.width // HYBRID_HEADS, "qkv_bias": False, "window": 0,
                "position": PartSpec("rotary", {"theta": HYBRID_THETA,
                                                "rotary_dim": self.width // HYBRID_HEADS,
                                                "max_position": 0})})
            toy_mixer = PartSpec("toy_decaying_sum", {"width": self.width, "decay": self.decay})
            layers = tuple(LayerSpec(
                prefix=f"blocks.{i}.", arrangement="prenorm",
                mixer=attention if i < self.attention_layers else toy_mixer,
                feed_forward=PartSpec("swiglu", {"hidden_size": self.width,
                                                 "intermediate_size": 2 * self.width}),
                mixer_norm=norm, feed_forward_norm=norm) for i in range(self.layers))
            return ModelSpec("ToyStateForCausalLM", self.width, self.vocab, 0, "embed.weight",
                             None, norm, "final_norm.", layers,
                             tuple(LayerCall(i) for i in range(self.layers)))

    register_architecture("ToyStateForCausalLM", ToyConfig)
    return ToyConfig


def undefine_toy():
    from from_scratch_inference_engine_b200.config import unregister_architecture
    from from_scratch_inference_engine_b200.parts import unregister_part
    unregister_architecture("ToyStateForCausalLM")
    unregister_part("mixer", "toy_decaying_sum")


def plain_toy(folder, ids):
    cfg = json.loads((folder / "config.json").read_text())
    w = plain.read_safetensors(folder / "model.safetensors")
    x = plain.embedding(w["embed.weight"], ids)
    for i in range(cfg["layers"]):
        p = f"blocks.{i}."
        y = plain.rms_norm(x, w[p + "mixer_norm.weight"], cfg["eps"])
        if i < cfg.get("attention_layers", 0):
            heads, hd, positions = HYBRID_HEADS, cfg["width"] // HYBRID_HEADS, list(range(len(ids)))
            q = plain.rope(plain.linear(y, w[p + "mixer.q_proj.weight"]), heads, hd, HYBRID_THETA, positions)
            k = plain.rope(plain.linear(y, w[p + "mixer.k_proj.weight"]), 1, hd, HYBRID_THETA, positions)
            v = plain.linear(y, w[p + "mixer.v_proj.weight"])
            x = x + plain.linear(plain.attention(q, k, v, heads, 1, hd), w[p + "mixer.o_proj.weight"])
        else:
            state = torch.zeros(cfg["width"], dtype=torch.float64)
            mixed = []
            for t in range(len(ids)):
                state = cfg["decay"] * state + y[t]
                mixed.append(state)
            x = x + plain.linear(torch.stack(mixed), w[p + "mixer.out.weight"])
        y = plain.rms_norm(x, w[p + "feed_forward_norm.weight"], cfg["eps"])
        x = x + plain.linear(plain.silu_mul(plain.linear(y, w[p + "feed_forward.gate_proj.weight"]),
                                            plain.linear(y, w[p + "feed_forward.up_proj.weight"])),
                             w[p + "feed_forward.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["final_norm.weight"], cfg["eps"]), w["embed.weight"])


@pytest.fixture()
def toy(tmp_path):
    config_class = define_toy()
    try:
        from from_scratch_inference_engine_b200 import write_random_model
        folder = write_random_model(tmp_path / "toy", config_class(40, 2, 77, 0.9, 1e-5),
                                    seed=4, std=0.2)
        yield folder
    finally:
        undefine_toy()


def test_toy_mixer_is_loaded_by_name_and_stepped_in_portions(toy):
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner, load_config
    assert type(load_config(toy)).__name__ == "ToyConfig"
    model = LoadedModel.from_pretrained(toy, dtype="float32", max_positions=256)
    runner = ModelRunner(model.model, model.runtime, page_size=16, num_pages=4, max_requests=2)
    assert runner.cache.groups == [] and runner.states[0].shape == (2, 40)
    requests = {k: helpers.random_ids(77, n, i) for i, (k, n) in
                enumerate({"a": 40, "b": 9, "c": 25, "d": 31}.items())}
    # two slots, four requests: slots are used again and must start from zero
    steps = helpers.trace_mixed(requests, seed=2, max_live=2)
    rows = helpers.run_trace_in_process(runner, steps)
    assert len(rows) == 105
    for (key, pos), row in rows.items():
        want = plain_toy(toy, requests[key])[pos].numpy()
        assert np.abs(row - want).max() < 1e-4 * max(1.0, np.abs(want).max())
    assert runner.cache.slots.num_free == 2


def test_toy_mixer_generates_through_the_scheduler(toy):
    from from_scratch_inference_engine_b200 import Engine, LoadedModel, SamplingParams
    model = LoadedModel.from_pretrained(toy, dtype="float32", max_positions=256)
    engine = Engine(model, block_size=16, num_blocks=4, max_batch=2, max_step_tokens=8)
    prompts = [helpers.random_ids(77, n, s) for n, s in ((13, 1), (5, 2), (20, 3))]
    ids = [engine.add_request(p, SamplingParams(temperature=0.0), 6) for p in prompts]
    engine.run_until_done()
    for rid, prompt in zip(ids, prompts):
        seq = list(prompt)
        for token in engine.output(rid):
            assert int(plain_toy(toy, seq)[-1].argmax()) == token
            seq.append(token)


def test_hybrid_of_attention_and_state_declines_prefix_sharing(tmp_path):
    """An attention layer's pages could be shared between requests with a common prefix; the
    state of the layer after it has no copy per page, so a request that skipped the shared
    tokens would start from a wrong state (and from what the slot's last owner left).  The
    cache manager therefore shares nothing for such a model, whatever the caller asks."""
    config_class = define_toy()
    try:
        from from_scratch_inference_engine_b200 import (Engine, LoadedModel, SamplingParams,
                                                        write_random_model)
        folder = write_random_model(tmp_path / "hybrid", config_class(32, 2, 61, 0.8, 1e-5, 1),
                                    seed=9, std=0.3)
        model = LoadedModel.from_pretrained(folder, dtype="float32", max_positions=256)
        engine = Engine(model, block_size=4, num_blocks=24, max_batch=1, max_step_tokens=8,
                        enable_prefix_cache=True)
        assert len(engine.runner.cache.groups) == 1 and not engine.runner.cache.prefix_enabled
        stem = helpers.random_ids(61, 13, 5)
        prompts = [stem + [3, 4], stem + [9], stem[:8] + [11, 12, 13]]
        for prompt in prompts:                  # one slot: each request inherits the last one's
            seq = list(prompt)
            for token in engine.generate(prompt, SamplingParams(temperature=0.0), 5):
                assert int(plain_toy(folder, seq)[-1].argmax()) == token
                seq.append(token)
        assert engine.prefix_hits() == 0
    finally:
        undefine_toy()
