"""Configuration and registry (no GPU)."""
import json

import pytest

from nncpu_b200.config import (AttentionSpec, GatedMlpSpec, architectures, config_from_dict,
                               load_config, register_architecture)
from nncpu_b200.errors import BadFormat, UnsupportedModel
from tiny import TINY, tiny_config


def test_every_size_comes_from_config_json():
    for name, d in TINY.items():
        c = tiny_config(name)
        spec = c.model_spec()
        assert len(spec.layers) == d["num_hidden_layers"] == len(spec.schedule)
        assert spec.hidden_size == d["hidden_size"] and spec.vocab_size == d["vocab_size"]
        a = spec.layers[0].mixer
        assert isinstance(a, AttentionSpec)
        assert (a.n_heads, a.n_kv_heads, a.head_dim) == (d["num_attention_heads"], d["num_key_value_heads"],
                                                         d["head_dim"])
        assert a.qk_norm.eps == d["rms_norm_eps"] == spec.layers[0].norm1.eps == spec.output.norm.eps
        assert a.position.theta == d["rope_theta"] and a.position.rotary_dim == d["head_dim"]
        assert abs(a.scale - d["head_dim"] ** -0.5) < 1e-12
        assert a.qkv_bias == d["attention_bias"]
        f = spec.layers[0].feed_forward
        assert isinstance(f, GatedMlpSpec) and f.intermediate_size == d["intermediate_size"]
        assert spec.output.tied == d["tie_word_embeddings"]
        assert spec.max_positions == d["max_position_embeddings"]


def test_defaults_follow_the_reference():
    d = dict(TINY["A"])
    for k in ("num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "max_position_embeddings",
              "tie_word_embeddings", "attention_bias", "eos_token_id"):
        d.pop(k)
    c = config_from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads          # load.rs:469
    assert c.head_dim == c.hidden_size // c.num_attention_heads     # load.rs:472-475
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0      # load.rs:476-481
    assert c.max_position_embeddings == 4096 and not c.tie_word_embeddings and not c.attention_bias
    assert c.model_spec().stop_token_ids == ()


def test_stop_tokens_int_or_list():
    assert tiny_config("A").model_spec().stop_token_ids == (255,)
    assert tiny_config("B").model_spec().stop_token_ids == (382, 383)


def test_windows_per_layer():
    assert tiny_config("A").windows() == [0, 0]
    assert tiny_config("C").windows() == [40, 0, 40, 0]
    spec = tiny_config("C").model_spec()
    assert [b.mixer.window for b in spec.layers] == [40, 0, 40, 0]
    # without layer_types the layers from max_window_layers on slide
    c = tiny_config("C", layer_types=None, max_window_layers=3)
    assert c.windows() == [0, 0, 0, 40]
    assert tiny_config("C", use_sliding_window=False).windows() == [0, 0, 0, 0]


def test_round_trip_through_config_json(tmp_path):
    for name in TINY:
        c = tiny_config(name)
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        assert load_config(tmp_path) == c


@pytest.mark.parametrize("change,err", [
    ({"num_key_value_heads": 3}, BadFormat),            # heads not a multiple of kv heads
    ({"head_dim": 15}, BadFormat),                      # odd head size
    ({"hidden_size": 0}, BadFormat),
    ({"num_hidden_layers": "two"}, BadFormat),
    ({"vocab_size": None}, BadFormat),
    ({"rms_norm_eps": -1.0}, BadFormat),
    ({"hidden_act": "gelu"}, UnsupportedModel),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, UnsupportedModel),
    ({"eos_token_id": 99999}, BadFormat),
    ({"layer_types": ["full_attention"]}, BadFormat),   # wrong count
    ({"layer_types": ["linear_attention", "full_attention"]}, UnsupportedModel),
])
def test_refusals(change, err):
    with pytest.raises(err):
        config_from_dict(dict(TINY["A"], **change))


def test_missing_basics_name_the_key():
    d = dict(TINY["A"])
    d.pop("intermediate_size")
    with pytest.raises(BadFormat, match="intermediate_size"):
        config_from_dict(d)


def test_registry():
    assert "Qwen3ForCausalLM" in architectures()
    with pytest.raises(UnsupportedModel, match="Qwen3ForCausalLM"):
        config_from_dict({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(BadFormat):
        config_from_dict({"hidden_size": 8})

    @register_architecture("ToyForTests")
    class Toy:
        @classmethod
        def from_dict(cls, d):
            return cls()
    assert isinstance(config_from_dict({"architectures": ["ToyForTests"]}), Toy)


def test_load_config_errors(tmp_path):
    with pytest.raises(BadFormat, match="does not exist"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(BadFormat, match="not JSON"):
        load_config(tmp_path)


def test_generation_config_adds_its_stop_tokens(tmp_path):
    d = dict(TINY["B"], eos_token_id=382)
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert load_config(tmp_path).eos_token_id == (382,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [383, 382], "temperature": 0.6}))
    cfg = load_config(tmp_path)
    assert cfg.eos_token_id == (382, 383) and cfg.model_spec().stop_token_ids == (382, 383)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5}))
    assert load_config(tmp_path).eos_token_id == (382, 5)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": ["x"]}))
    with pytest.raises(BadFormat, match="generation_config"):
        load_config(tmp_path)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 99999}))
    with pytest.raises(BadFormat, match="outside the vocabulary"):
        load_config(tmp_path)


def test_written_config_holds_no_key_without_a_value():
    for name in TINY:
        d = tiny_config(name).to_dict()
        assert all(v is not None for v in d.values()), [k for k, v in d.items() if v is None]
    assert "sliding_window" in tiny_config("C").to_dict() and "sliding_window" not in tiny_config("A").to_dict()
