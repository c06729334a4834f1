"""Configuration: the typed Qwen2 config from config.json keys, the registries, the model description."""
import json
import os

import pytest

import helpers
import vipera_rs_b200  # noqa: F401
from vipera_rs_b200 import errors
from vipera_rs_b200.config import (ARCHITECTURES, MIXERS, ModelSpec, Qwen2Config, ScheduleEntry, architecture_of,
                                   load_config, qwen2_model_spec)
from vipera_rs_b200 import parts  # noqa: F401  (registers the built-in kinds)


def test_reads_every_size_from_config_json(tmp_path):
    for name, raw in helpers.CONFIGS.items():
        (tmp_path / name).mkdir()
        with open(tmp_path / name / "config.json", "w") as handle:
            json.dump(raw, handle)
        arch, config = load_config(str(tmp_path / name))
        assert arch.name == "Qwen2ForCausalLM"
        assert config.num_hidden_layers == raw["num_hidden_layers"]
        assert config.hidden_size == raw["hidden_size"]
        assert config.num_key_value_heads == raw["num_key_value_heads"]
        assert config.head_dim == raw.get("head_dim", raw["hidden_size"] // raw["num_attention_heads"])
        assert config.vocab_size == raw["vocab_size"]
        assert config.rms_norm_eps == raw["rms_norm_eps"] and config.rope_theta == raw["rope_theta"]
        assert config.tie_word_embeddings == raw["tie_word_embeddings"]
        assert Qwen2Config.from_dict(config.to_dict()) == config


def test_defaults_follow_the_reference():
    config = Qwen2Config.from_dict({"num_hidden_layers": 1, "hidden_size": 64, "num_attention_heads": 4,
                                    "intermediate_size": 32, "vocab_size": 10})
    assert config.num_key_value_heads == 4          # defaults to the number of heads
    assert config.head_dim == 16
    assert config.rms_norm_eps == 1e-6 and config.rope_theta == 10000.0
    assert config.tie_word_embeddings is False and config.use_sliding_window is False


@pytest.mark.parametrize("change,error", [
    ({"hidden_size": None}, errors.UnsupportedError),                 # a required key is missing
    ({"num_attention_heads": 5}, errors.InvalidArgumentError),        # hidden not a multiple of heads
    ({"num_key_value_heads": 3}, errors.InvalidArgumentError),        # heads not a multiple of kv heads
    ({"head_dim": 15}, errors.InvalidArgumentError),                  # odd head size
    ({"num_hidden_layers": 0}, errors.InvalidArgumentError),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, errors.UnsupportedError),
    ({"hidden_act": "gelu"}, errors.UnsupportedError),
    ({"use_sliding_window": True, "sliding_window": None}, errors.InvalidArgumentError),
    ({"rms_norm_eps": 0.0}, errors.InvalidArgumentError),
])
def test_rejects_bad_configurations(change, error):
    raw = dict(helpers.TINY_A)
    for key, value in change.items():
        if value is None and key in ("hidden_size",):
            raw.pop(key)
        else:
            raw[key] = value
    with pytest.raises(error):
        Qwen2Config.from_dict(raw)


def test_unknown_architecture_lists_the_registered_ones():
    with pytest.raises(errors.UnsupportedError) as info:
        architecture_of({"architectures": ["LlamaForCausalLM"]})
    assert "Qwen2ForCausalLM" in str(info.value)
    with pytest.raises(errors.UnsupportedError):
        architecture_of({})
    assert "Qwen2ForCausalLM" in ARCHITECTURES.names()
    assert "gqa_attention" in MIXERS


def test_model_spec_is_layer_by_layer():
    config = Qwen2Config.from_dict(helpers.TINY_B)
    spec = qwen2_model_spec(config)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    windows = [layer.parts["mixer"].params["window"] for layer in spec.layers]
    assert windows == [None, 80, 80]                # layers from max_window_layers up see a window
    assert spec.head_name == "lm_head.weight"
    tied = qwen2_model_spec(Qwen2Config.from_dict(helpers.TINY_A))
    assert tied.head_name is None
    assert tied.layers[0].parts["mixer"].params["position"].params["theta"] == 10000.0
    assert spec.layers[0].part_prefix("mixer") == "model.layers.0.self_attn"


def test_schedule_validation():
    spec = qwen2_model_spec(Qwen2Config.from_dict(helpers.TINY_A))

    def with_schedule(schedule):
        return ModelSpec(**{**spec.__dict__, "schedule": schedule})

    with_schedule([ScheduleEntry(0, 0), ScheduleEntry(0, 1), ScheduleEntry(1, 0, writes_cache=False)]).validate()
    with pytest.raises(errors.InvalidArgumentError):
        with_schedule([ScheduleEntry(0, 0), ScheduleEntry(1, 0)]).validate()        # two writers of one slot
    with pytest.raises(errors.InvalidArgumentError):
        with_schedule([ScheduleEntry(0, 0, writes_cache=False)]).validate()          # read before written
    with pytest.raises(errors.InvalidArgumentError):
        with_schedule([ScheduleEntry(5, 0)]).validate()


def test_parameter_count_matches_the_reference_contract():
    """1,543,714,304 parameters for the Qwen2.5-1.5B shape
    (specs/001-vipera-rs-engine/contracts/cli.md:31)."""
    config = Qwen2Config.from_dict({
        "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
        "intermediate_size": 8960, "vocab_size": 151936, "tie_word_embeddings": True})
    assert config.parameter_count() == 1543714304
    assert config.kv_bytes_per_token(2) == 28672   # crates/vipera-backend-cpu/src/model.rs:1406
