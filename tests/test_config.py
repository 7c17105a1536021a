"""Configuration parsing and the architecture registry (no GPU). The table of
refusals follows crates/models/qwen/src/forward.rs:461-557 and its tests at
:3004-3282."""
import json

import pytest

from conftest import TINY_A, TINY_B, TINY_C
from metallix_b200.config import (ConfigError, Qwen3Config, family_by_kind, parse_config, read_config,
                                  resolve)

QWEN3_0_6B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
                  attention_bias=False, num_hidden_layers=28, hidden_size=1024,
                  intermediate_size=3072, vocab_size=151936, num_attention_heads=16,
                  num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                  rms_norm_eps=1e-6, rope_theta=1000000, tie_word_embeddings=True,
                  sliding_window=None, use_sliding_window=False, max_window_layers=28,
                  rope_scaling=None, eos_token_id=151645)


def test_parses_the_0_6b_layout():
    config = Qwen3Config.from_dict(QWEN3_0_6B)
    assert config.num_hidden_layers == 28 and config.head_dim == 128
    assert config.num_attention_heads * config.head_dim == 2048 != config.hidden_size
    assert config.tie_word_embeddings and config.eos_token_ids == (151645,)
    assert config.kv_bytes_per_token(2) == 28 * 2 * 8 * 128 * 2  # forward.rs:622-638
    assert config.parameter_count() == 596_049_920


def test_defaults():
    raw = {k: v for k, v in TINY_A.items() if k not in ("rms_norm_eps", "rope_theta", "tie_word_embeddings")}
    config = Qwen3Config.from_dict(raw)
    assert config.rms_norm_eps == pytest.approx(1e-6)
    assert config.rope_theta == 1_000_000.0       # forward.rs:2659-2661
    assert config.tie_word_embeddings is False    # forward.rs:2606-2607


@pytest.mark.parametrize("change, kind", [
    ({"model_type": "llama"}, "UnsupportedModelType"),
    ({"model_type": "qwen3", "use_bidirectional_attention": True}, "UnsupportedModelType"),
    ({"attention_bias": True}, "UnsupportedBiasLayout"),
    ({"mlp_bias": True}, "UnsupportedBiasLayout"),
    ({"hidden_act": "gelu"}, "UnsupportedActivation"),
    ({"hidden_act": None}, "UnsupportedActivation"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "UnsupportedRopeScaling"),
    ({"rope_parameters": {"rope_type": "yarn", "rope_theta": 1e6}}, "UnsupportedRopeScaling"),
    ({"rope_parameters": {"rope_type": "default", "rope_theta": 1e4, "factor": 2}}, "UnsupportedRopeScaling"),
    ({"rope_parameters": {"rope_type": "default", "rope_theta": 5e5}}, "ConflictingRopeTheta"),
    ({"use_sliding_window": True, "sliding_window": 64}, "UnsupportedSlidingWindow"),
    ({"quantization": {"group_size": 64, "bits": 4}}, "UnsupportedQuantization"),
    ({"quantization_config": {"quant_method": "fp8"}}, "UnsupportedQuantization"),
    ({"num_hidden_layers": 0}, "MissingDimension"),
    ({"head_dim": None}, "MissingDimension"),
    ({"vocab_size": 0}, "MissingDimension"),
    ({"head_dim": 15}, "OddHeadDimension"),
    ({"head_dim": 65536}, "HeadDimensionTooLarge"),
    ({"num_attention_heads": 5, "num_key_value_heads": 2}, "InvalidGroupedQueryLayout"),
    ({"rms_norm_eps": 0.0}, "InvalidRmsNormEpsilon"),
    ({"rms_norm_eps": -1e-6}, "InvalidRmsNormEpsilon"),
    ({"rope_theta": 0.0}, "InvalidRopeTheta"),
    ({"rope_theta": 1e39}, "InvalidRopeTheta"),
])
def test_refusals(change, kind):
    raw = dict(TINY_A, **change)
    with pytest.raises(ConfigError) as error:
        Qwen3Config.from_dict(raw)
    assert error.value.kind == kind


def test_missing_hidden_act_is_refused():
    raw = {k: v for k, v in TINY_A.items() if k != "hidden_act"}
    with pytest.raises(ConfigError) as error:
        Qwen3Config.from_dict(raw)
    assert error.value.kind == "UnsupportedActivation"   # forward.rs:2604-2605,472


def test_rope_parameters_supply_theta():
    raw = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    raw["rope_parameters"] = {"rope_type": "default", "rope_theta": 12345.0}
    assert Qwen3Config.from_dict(raw).rope_theta == 12345.0
    raw["rope_theta"] = 12345.0
    assert Qwen3Config.from_dict(raw).rope_theta == 12345.0


def test_ignored_window_key():
    raw = dict(TINY_A, sliding_window=32768, use_sliding_window=False)  # forward.rs:518-528
    assert Qwen3Config.from_dict(raw).hidden_size == 64


def test_malformed_json():
    with pytest.raises(ConfigError) as error:
        Qwen3Config.parse("{not json")
    assert error.value.kind == "Json"
    with pytest.raises(ConfigError):
        Qwen3Config.parse("[1, 2]")


def test_round_trip_through_to_dict():
    for raw in (TINY_A, TINY_B, QWEN3_0_6B):
        config = Qwen3Config.from_dict(raw)
        assert Qwen3Config.parse(json.dumps(config.to_dict())) == config


def test_registry_by_every_name():
    assert resolve(TINY_A).config_class is Qwen3Config
    assert resolve({"model_type": "qwen3"}).config_class is Qwen3Config
    assert resolve({"architectures": ["Qwen3ForCausalLM"]}).config_class is Qwen3Config
    assert family_by_kind("qwen").architecture == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError) as error:
        resolve({"architectures": ["GemmaForCausalLM"], "model_type": "gemma"})
    assert "GemmaForCausalLM" in str(error.value) and "gemma" in str(error.value)
    assert isinstance(parse_config(TINY_B), Qwen3Config)


def test_read_config_merges_generation_eos(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, eos_token_id=7)))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 9]}))
    assert read_config(str(tmp_path)).eos_token_ids == (7, 9)
    with pytest.raises(ConfigError):
        read_config(str(tmp_path / "missing"))


def test_model_spec_is_data():
    spec = Qwen3Config.from_dict(TINY_B).to_model_spec()
    assert len(spec.layers) == 3 and [run.layer for run in spec.order] == [0, 1, 2]
    mixer = spec.layers[1].mixer
    assert mixer.kind == "gqa_attention" and mixer["num_heads"] == 6 and mixer["num_kv_heads"] == 2
    assert mixer["scale"] == pytest.approx(32 ** -0.5)
    assert mixer["position"].kind == "rope_half" and mixer["position"]["theta"] == 1e6
    assert mixer["q_norm"]["weight"] == "model.layers.1.self_attn.q_norm.weight"
    assert spec.head["weight"] == "lm_head.weight"
    assert Qwen3Config.from_dict(TINY_A).to_model_spec().head["weight"] == "model.embed_tokens.weight"


def test_no_size_stands_in_code():
    """Every size of the spec changes when the configuration changes."""
    a = Qwen3Config.from_dict(TINY_A).to_model_spec()
    b = Qwen3Config.from_dict(TINY_B).to_model_spec()
    c = Qwen3Config.from_dict(TINY_C).to_model_spec()
    for key in ("hidden_size", "num_heads", "head_dim", "scale"):
        assert a.layers[0].mixer[key] != b.layers[0].mixer[key]
    assert a.layers[0].mixer["num_kv_heads"] != c.layers[0].mixer["num_kv_heads"]
    assert a.layers[0].mixer["num_heads"] // a.layers[0].mixer["num_kv_heads"] != \
        b.layers[0].mixer["num_heads"] // b.layers[0].mixer["num_kv_heads"]
    assert a.layers[0].feed_forward["intermediate_size"] != b.layers[0].feed_forward["intermediate_size"]
    assert a.layers[0].mixer_norm["eps"] != b.layers[0].mixer_norm["eps"]
    assert a.vocab_size != b.vocab_size and a.max_positions != b.max_positions
