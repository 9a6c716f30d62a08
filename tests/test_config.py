"""Configuration and registry (reference behaviour: tests/cpp/test_safetensors.cpp:105-140)."""

import json

import pytest

from from_scratch_inference_engine_b200.config import (ConfigError, LayerCall, Qwen2Config,
                                                        config_from_dict, load_config,
                                                        register_architecture,
                                                        registered_architectures,
                                                        unregister_architecture)
from helpers import TINY


def base(**extra):
    data = dict(model_type="qwen2", hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                intermediate_size=176, vocab_size=256)
    data.update(extra)
    return data


def test_defaults_and_derived_values():
    c = Qwen2Config.from_dict(base())
    assert c.num_key_value_heads == 4            # defaults to the head count
    assert c.head_dim == 16                      # hidden / heads
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6
    assert c.attention_qkv_bias is True          # model_type qwen2 forces the bias
    assert c.tie_word_embeddings is False and c.max_position_embeddings == 0


def test_explicit_head_dim_and_bias_of_other_model_types():
    c = Qwen2Config.from_dict(base(head_dim=32, model_type="other",
                                   architectures=["Qwen2ForCausalLM"]))
    assert c.head_dim == 32 and c.q_width == 128 and c.attention_qkv_bias is False
    c = Qwen2Config.from_dict(base(model_type="other", attention_bias=True))
    assert c.attention_qkv_bias is True


@pytest.mark.parametrize("bad", [
    dict(num_attention_heads=0), dict(num_key_value_heads=3), dict(head_dim=15),
    dict(hidden_act="gelu"), dict(vocab_size=0), dict(rope_theta=-1.0),
    dict(use_sliding_window=True, sliding_window=0),
    dict(use_sliding_window=True, sliding_window=8, max_window_layers=5),
    dict(rope_scaling={"type": "yarn", "factor": 4.0}),
])
def test_invalid_values_are_refused(bad):
    with pytest.raises(ConfigError):
        Qwen2Config.from_dict(base(**bad))


def test_missing_key_is_named():
    data = base()
    del data["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        Qwen2Config.from_dict(data)


def test_registry_resolves_by_architecture_then_model_type(tmp_path):
    assert "Qwen2ForCausalLM" in registered_architectures()
    assert isinstance(config_from_dict(base()), Qwen2Config)          # via model_type
    assert isinstance(config_from_dict(base(architectures=["Qwen2ForCausalLM"], model_type="x")),
                      Qwen2Config)
    with pytest.raises(ConfigError, match="NopeForCausalLM.*registered"):
        config_from_dict(base(architectures=["NopeForCausalLM"]))
    with pytest.raises(ConfigError, match="names no architecture"):
        config_from_dict({k: v for k, v in base().items() if k != "model_type"})
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(tmp_path)
    with pytest.raises(ConfigError, match="cannot read"):
        load_config(tmp_path / "absent")


def test_registering_another_architecture():
    class Other:
        @classmethod
        def from_dict(cls, data):
            return cls()

        def to_dict(self):
            return {}

        def build_spec(self):
            raise NotImplementedError
    register_architecture("OtherForCausalLM", Other)
    try:
        assert isinstance(config_from_dict({"architectures": ["OtherForCausalLM"]}), Other)
    finally:
        unregister_architecture("OtherForCausalLM")
    with pytest.raises(TypeError):
        register_architecture("Broken", object)


def test_round_trip_through_config_json(tmp_path):
    for entry in TINY.values():
        c = config_from_dict(entry["config"])
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        assert load_config(tmp_path) == c


def test_spec_is_data_layer_by_layer():
    c = config_from_dict(TINY["C"]["config"])
    spec = c.build_spec()
    windows = [layer.mixer.params["window"] for layer in spec.layers]
    assert windows == [0, 21, 21]                       # max_window_layers = 1
    assert spec.head_name == "lm_head.weight"
    assert config_from_dict(TINY["A"]["config"]).build_spec().head_name is None
    assert [c.layer for c in spec.schedule] == [0, 1, 2]
    assert spec.resolved_schedule() == [(0, 0, True), (1, 1, True), (2, 2, True)]


def test_schedule_checks():
    import dataclasses
    spec = config_from_dict(TINY["A"]["config"]).build_spec()
    twice = dataclasses.replace(spec, schedule=(LayerCall(0), LayerCall(1), LayerCall(0)))
    assert twice.resolved_schedule() == [(0, 0, True), (1, 1, True), (0, 2, True)]
    shared = dataclasses.replace(spec, schedule=(LayerCall(0), LayerCall(1, cache=0,
                                                                         writes_cache=False)))
    assert shared.resolved_schedule() == [(0, 0, True), (1, 0, False)]
    with pytest.raises(ValueError, match="before any call has written"):
        dataclasses.replace(spec, schedule=(LayerCall(0, cache=1, writes_cache=False),
                                            LayerCall(1))).resolved_schedule()
    with pytest.raises(ValueError, match="written twice"):
        dataclasses.replace(spec, schedule=(LayerCall(0), LayerCall(1, cache=0))
                            ).resolved_schedule()
    with pytest.raises(ValueError, match="names layer"):
        dataclasses.replace(spec, schedule=(LayerCall(5),)).resolved_schedule()
