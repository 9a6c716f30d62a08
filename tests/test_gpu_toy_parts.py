"""Toy parts defined in the test - a feed-forward with routing and a position encoding of
another kind - are registered, built from a configuration, loaded by name and stepped through
the cache and the scheduler without a change to the package (the stateful toy mixer has its
own file).  They show the generality of the part interfaces; they are not a model of anyone's."""

import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu


def define():
    from from_scratch_inference_engine_b200.config import (LayerCall, LayerSpec, ModelSpec,
                                                            PartSpec, register_architecture)
    from from_scratch_inference_engine_b200.parts import Part, register_part
    from from_scratch_inference_engine_b200.weights import TensorSpec

    @register_part("feed_forward", "toy_top1_experts")
    class Top1Experts(Part):
        """Router logits in float32, the token goes to its best expert (a two-matrix ReLU MLP),
        the expert's output is scaled by the router's softmax weight of that expert."""

        def __init__(self, prefix, width, inner, experts):
            self.prefix, self.width, self.inner, self.experts = prefix, width, inner, experts

        def tensor_specs(self):
            specs = [TensorSpec(self.prefix + "router.weight", (self.experts, self.width))]
            for e in range(self.experts):
                specs += [TensorSpec(self.prefix + f"experts.{e}.up.weight", (self.inner, self.width)),
                          TensorSpec(self.prefix + f"experts.{e}.down.weight", (self.width, self.inner))]
            return specs

        def bind(self, tensors, runtime):
            self.runtime = runtime
            self.router = tensors[self.prefix + "router.weight"].float()
            self.up = [tensors[self.prefix + f"experts.{e}.up.weight"] for e in range(self.experts)]
            self.down = [tensors[self.prefix + f"experts.{e}.down.weight"] for e in range(self.experts)]

        def forward(self, ctx, y):
            logits = y.float() @ self.router.T                       # routing in 32-bit
            weight, choice = torch.softmax(logits, -1).max(-1)
            out = torch.zeros_like(y)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    hidden = torch.relu(self.runtime.linear(y[rows].contiguous(), self.up[e], None))
                    part = self.runtime.linear(hidden, self.down[e], None)
                    out[rows] = (part.float() * weight[rows, None]).to(y.dtype)
            return out

    @register_part("position", "toy_learned_rotary")
    class LearnedAngles(Part):
        """Rotary pairs whose angles come from a stored table [max_position, rotary_dim / 2]
        instead of a formula: the mixer's kernel is the same, only the cos/sin table differs."""

        def __init__(self, prefix, rotary_dim, max_position):
            self.prefix, self.rotary_dim, self.max_position = prefix, rotary_dim, max_position

        def tensor_specs(self):
            return [TensorSpec(self.prefix + "angles", (self.max_position, self.rotary_dim // 2),
                               role="vector")]

        def bind(self, tensors, runtime):
            angles = tensors[self.prefix + "angles"].double() * 3.0
            self.table = torch.cat([angles.cos(), angles.sin()], 1).float().contiguous()

    @dataclass(frozen=True)
    class ToyPartsConfig:
        width: int
        vocab: int
        heads: int
        head_dim: int
        experts: int

        @classmethod
        def from_dict(cls, d):
            return cls(d["width"], d["vocab"], d["heads"], d["head_dim"], d["experts"])

        def to_dict(self):
            return {"architectures": ["ToyPartsForCausalLM"], "width": self.width, "vocab": self.vocab,
                    "heads": self.heads, "head_dim": self.head_dim, "experts": self.experts}

        def build_spec(self):
            norm = PartSpec("rmsnorm", {"width": self.width, "eps": 1e-5})
            attention = PartSpec("gqa_attention", {
                "hidden_size": self.width, "num_heads": self.heads, "num_kv_heads": self.heads,
                "head_dim": self.head_dim, "qkv_bias": False, "window": 0,
                "position": PartSpec("toy_learned_rotary", {"rotary_dim": self.head_dim // 2,
                                                            "max_position": 96})})
            routed = PartSpec("toy_top1_experts", {"width": self.width, "inner": 2 * self.width,
                                                   "experts": self.experts})
            dense = PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": 72})
            layers = tuple(LayerSpec(prefix=f"layers.{i}.", arrangement="prenorm", mixer=attention,
                                     feed_forward=routed if i % 2 == 0 else dense,
                                     mixer_norm=norm, feed_forward_norm=norm) for i in range(3))
            return ModelSpec("ToyPartsForCausalLM", self.width, self.vocab, 96, "embed.weight",
                             "head.weight", norm, "final_norm.", layers,
                             tuple(LayerCall(i) for i in range(3)))

    register_architecture("ToyPartsForCausalLM", ToyPartsConfig)
    return ToyPartsConfig


def undefine():
    from from_scratch_inference_engine_b200.config import unregister_architecture
    from from_scratch_inference_engine_b200.parts import unregister_part
    unregister_architecture("ToyPartsForCausalLM")
    unregister_part("feed_forward", "toy_top1_experts")
    unregister_part("position", "toy_learned_rotary")


def plain_forward(folder, ids):
    cfg = json.loads((folder / "config.json").read_text())
    w = plain.read_safetensors(folder / "model.safetensors")
    heads, hd, rot = cfg["heads"], cfg["head_dim"], cfg["head_dim"] // 2
    x = plain.embedding(w["embed.weight"], ids)
    n = len(ids)

    def rotate(t, p):
        angles = w[p + "mixer.angles"][:n] * 3.0                     # [n, rot / 2]
        c, s = angles.cos()[:, None, :], angles.sin()[:, None, :]
        th = t.reshape(n, heads, hd)
        a, b, rest = th[..., :rot // 2], th[..., rot // 2:rot], th[..., rot:]
        return torch.cat([a * c - b * s, b * c + a * s, rest], -1).reshape(n, heads * hd)
    for i in range(3):
        p = f"layers.{i}."
        y = plain.rms_norm(x, w[p + "mixer_norm.weight"], 1e-5)
        q = rotate(plain.linear(y, w[p + "mixer.q_proj.weight"]), p)
        k = rotate(plain.linear(y, w[p + "mixer.k_proj.weight"]), p)
        v = plain.linear(y, w[p + "mixer.v_proj.weight"])
        x = x + plain.linear(plain.attention(q, k, v, heads, heads, hd), w[p + "mixer.o_proj.weight"])
        y = plain.rms_norm(x, w[p + "feed_forward_norm.weight"], 1e-5)
        if i % 2 == 0:
            probs = torch.softmax(plain.linear(y, w[p + "feed_forward.router.weight"]), -1)
            weight, choice = probs.max(-1)
            out = torch.zeros_like(y)
            for t in range(n):
                e = int(choice[t])
                hidden = torch.relu(plain.linear(y[t:t + 1], w[p + f"feed_forward.experts.{e}.up.weight"]))
                out[t] = plain.linear(hidden, w[p + f"feed_forward.experts.{e}.down.weight"])[0] * weight[t]
            x = x + out
        else:
            x = x + plain.linear(plain.silu_mul(plain.linear(y, w[p + "feed_forward.gate_proj.weight"]),
                                                plain.linear(y, w[p + "feed_forward.up_proj.weight"])),
                                 w[p + "feed_forward.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["final_norm.weight"], 1e-5), w["head.weight"])


@pytest.fixture()
def toy(tmp_path):
    config_class = define()
    try:
        from from_scratch_inference_engine_b200 import write_random_model
        yield write_random_model(tmp_path / "toy", config_class(48, 90, 3, 16, 3), seed=6, std=0.25,
                                 dtype=torch.float32)
    finally:
        undefine()


def test_routed_feed_forward_and_learned_positions_step_through_the_engine(toy):
    from from_scratch_inference_engine_b200 import LoadedModel, ModelRunner
    model = LoadedModel.from_pretrained(toy, dtype="float32", max_positions=96)
    kinds = [type(b.feed_forward).__name__ for b in model.model.blocks]
    assert kinds == ["Top1Experts", "SwiGluMlp", "Top1Experts"]       # chosen layer by layer
    runner = ModelRunner(model.model, model.runtime, page_size=8, num_pages=24, max_requests=3)
    assert not runner.cuda_graphs          # the routed part reads the device: nothing is captured
    requests = {k: helpers.random_ids(90, n, i) for i, (k, n) in
                enumerate({"a": 60, "b": 17, "c": 41}.items())}
    rows = helpers.run_trace_in_process(runner, helpers.trace_mixed(requests, seed=5, max_live=3))
    assert len(rows) == 118
    want = {k: plain_forward(toy, ids).numpy() for k, ids in requests.items()}
    worst = max(np.abs(row - want[k][pos]).max() for (k, pos), row in rows.items())
    assert worst < 2e-4, worst
