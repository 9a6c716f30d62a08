"""Safetensors container, weight checks and the random-weights mode
(reference behaviour: tests/cpp/test_safetensors.cpp:41-103)."""

import json
import struct

import numpy as np
import pytest
import torch

from from_scratch_inference_engine_b200.config import config_from_dict
from from_scratch_inference_engine_b200.parts import tensor_specs
from from_scratch_inference_engine_b200.weights import (SafeTensorsError, TensorSpec, WeightError,
                                                         check_tensors, load_checkpoint,
                                                         load_file, parse, random_tensors,
                                                         save_file, serialize, standard_normal,
                                                         to_runtime_dtype, write_random_model)
from helpers import TINY
import plain_qwen2 as plain


def container(header: dict, data: bytes = b"") -> bytes:
    text = json.dumps(header).encode()
    return struct.pack("<Q", len(text)) + text + data


def test_round_trip_keeps_dtypes_and_values(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
               "d": torch.randn(4).to(torch.float16)}
    save_file(tensors, tmp_path / "x.safetensors")
    back = load_file(tmp_path / "x.safetensors")
    assert set(back) == set(tensors)
    for name, tensor in tensors.items():
        assert back[name].dtype == tensor.dtype and torch.equal(back[name], tensor)
    # the plain reader of the tests sees the same numbers
    save_file({k: v for k, v in tensors.items() if k != "c"}, tmp_path / "y.safetensors")
    other = plain.read_safetensors(tmp_path / "y.safetensors")
    assert torch.equal(other["b"].float(), tensors["b"].float())


def test_f32_and_bf16_parse_like_the_reference():
    data = struct.pack("<2f", 1.5, -2.0) + struct.pack("<2H", 0x3F80, 0xC000)   # bf16 1.0, -2.0
    header = {"__metadata__": {"format": "pt"},
              "f": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
              "b": {"dtype": "BF16", "shape": [1, 2], "data_offsets": [8, 12]}}
    out = parse(container(header, data))
    assert out["f"].tolist() == [1.5, -2.0]
    assert out["b"].float().tolist() == [[1.0, -2.0]] and out["b"].dtype is torch.bfloat16


@pytest.mark.parametrize("blob,message", [
    (b"\x01\x02", "smaller than the 8-byte"),
    (struct.pack("<Q", 1 << 60) + b"{}", "header length exceeds"),
    (struct.pack("<Q", 5) + b"{not}", "invalid header JSON"),
    (container({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8),
     "out of range"),
    (container({"t": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}, b"\0" * 4),
     "negative dimension"),
    (container({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8),
     "byte count does not match"),
    (container({"t": {"dtype": "F32", "shape": [2]}}, b"\0" * 8), "malformed header entry"),
    (container({"t": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}, b"\0" * 8),
     "unsupported dtype"),
    (container({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12),
     "overlapping"),
])
def test_hardening(blob, message):
    with pytest.raises(SafeTensorsError, match=message):
        parse(blob)


def test_duplicate_name_and_missing_file(tmp_path):
    text = b'{"t":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},' \
           b'"t":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'
    with pytest.raises(SafeTensorsError, match="duplicate"):
        parse(struct.pack("<Q", len(text)) + text + b"\0" * 8)
    with pytest.raises(SafeTensorsError, match="cannot open"):
        load_file(tmp_path / "absent.safetensors")


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    specs = [TensorSpec("a", (2, 3)), TensorSpec("b", (4,)), TensorSpec("c", (5,)),
             TensorSpec("opt", (1,), optional=True)]
    tensors = {"a": torch.zeros(3, 2), "c": torch.zeros(5), "zzz": torch.zeros(1),
               "yyy": torch.zeros(1)}
    with pytest.raises(WeightError) as error:
        check_tensors(specs, tensors)
    text = str(error.value)
    assert "missing (1): b" in text
    assert "unexpected (2): yyy, zzz" in text
    assert "a: expected [2, 3], found [3, 2]" in text
    check_tensors(specs, {"a": torch.zeros(2, 3), "b": torch.zeros(4), "c": torch.zeros(5)})


def test_tied_head_stored_twice_must_equal_the_embedding():
    spec = config_from_dict(TINY["A"]["config"]).build_spec()
    specs = tensor_specs(spec)
    tensors = random_tensors(specs, 0)
    check_tensors(specs, tensors)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    check_tensors(specs, tensors)
    tensors["lm_head.weight"] = tensors["lm_head.weight"] + 1
    with pytest.raises(WeightError, match="must equal"):
        check_tensors(specs, tensors)
    untied = tensor_specs(config_from_dict(TINY["B"]["config"]).build_spec())
    with pytest.raises(WeightError, match="missing.*lm_head.weight"):
        check_tensors(untied, {k: v for k, v in random_tensors(untied, 0).items()
                               if k != "lm_head.weight"})


def test_model_tensor_names_are_the_checkpoint_names():
    c = config_from_dict(TINY["B"]["config"])
    names = {s.name: s.shape for s in tensor_specs(c.build_spec())}
    assert names["model.embed_tokens.weight"] == (384, 192)
    assert names["model.layers.2.self_attn.q_proj.weight"] == (192, 192)
    assert names["model.layers.0.self_attn.k_proj.bias"] == (32,)
    assert names["model.layers.1.self_attn.o_proj.weight"] == (192, 192)
    assert names["model.layers.1.mlp.gate_proj.weight"] == (512, 192)
    assert names["model.layers.1.mlp.down_proj.weight"] == (192, 512)
    assert names["model.layers.0.input_layernorm.weight"] == (192,)
    assert names["model.layers.0.post_attention_layernorm.weight"] == (192,)
    assert names["model.norm.weight"] == (192,) and names["lm_head.weight"] == (384, 192)
    d = {s.name: s.shape for s in
         tensor_specs(config_from_dict(TINY["D"]["config"]).build_spec())}
    assert d["model.layers.0.self_attn.o_proj.weight"] == (96, 128)     # [hidden, q width]


def test_dtype_rule():
    matrix, vector = TensorSpec("m", (2, 2)), TensorSpec("v", (2,), role="vector")
    table = TensorSpec("t", (2,), role="table")
    f32, b16 = torch.ones(2, 2), torch.ones(2, 2, dtype=torch.bfloat16)
    assert to_runtime_dtype(f32, matrix, torch.bfloat16).dtype is torch.bfloat16
    assert to_runtime_dtype(b16, matrix, torch.float32).dtype is torch.float32
    assert to_runtime_dtype(torch.ones(2), vector, torch.bfloat16).dtype is torch.float32
    assert to_runtime_dtype(torch.ones(2).bfloat16(), vector, torch.bfloat16).dtype \
        is torch.bfloat16
    assert to_runtime_dtype(torch.ones(2, dtype=torch.int64), table, torch.bfloat16).dtype \
        is torch.int32


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    c = config_from_dict(TINY["A"]["config"])
    folder = write_random_model(tmp_path / "m", c, seed=0, std=0.02)
    assert json.loads((folder / "config.json").read_text())["architectures"] == \
        ["Qwen2ForCausalLM"]
    tensors = load_checkpoint(folder)
    check_tensors(tensor_specs(c.build_spec()), tensors)
    assert all(t.dtype is torch.bfloat16 for t in tensors.values())
    again = load_checkpoint(write_random_model(tmp_path / "n", c, seed=0, std=0.02))
    assert all(torch.equal(tensors[k], again[k]) for k in tensors)
    other = load_checkpoint(write_random_model(tmp_path / "o", c, seed=1, std=0.02))
    assert not torch.equal(tensors["model.norm.weight"], other["model.norm.weight"])
    gain = tensors["model.norm.weight"].float()
    assert abs(gain.mean().item() - 1.0) < 0.02          # gains are 1 + N(0, std)
    w = tensors["model.layers.0.mlp.up_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002


def test_standard_normal_is_keyed_by_seed_and_name():
    a = standard_normal(3, "x", 10000)
    assert np.array_equal(a[:100], standard_normal(3, "x", 100))
    assert not np.array_equal(a[:100], standard_normal(3, "y", 100))
    assert abs(a.mean()) < 0.05 and abs(a.std() - 1.0) < 0.05


def test_sharded_checkpoint_is_read_through_its_index(tmp_path):
    c = config_from_dict(TINY["A"]["config"])
    folder = write_random_model(tmp_path / "m", c, seed=0, std=0.02)
    whole = load_checkpoint(folder)
    names = sorted(whole)
    first, second = names[:len(names) // 2], names[len(names) // 2:]
    save_file({n: whole[n] for n in first}, folder / "model-00001-of-00002.safetensors")
    save_file({n: whole[n] for n in second}, folder / "model-00002-of-00002.safetensors")
    index = {"weight_map": {**{n: "model-00001-of-00002.safetensors" for n in first},
                            **{n: "model-00002-of-00002.safetensors" for n in second}}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    (folder / "model.safetensors").unlink()
    shards = load_checkpoint(folder)
    assert set(shards) == set(whole) and all(torch.equal(shards[n], whole[n]) for n in whole)
    index["weight_map"]["ghost.weight"] = "model-00002-of-00002.safetensors"
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(WeightError, match="ghost.weight"):
        load_checkpoint(folder)
