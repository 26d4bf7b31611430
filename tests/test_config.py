"""Typed configuration and the architecture registry."""

import json

import pytest

from conftest import TINY, tiny_raw
from starter_b200.config import ConfigError, architecture_names, config_from_dict, load_config, save_config
from starter_b200.models.qwen3 import Qwen3Config


def test_fields_come_from_config_json():
    cfg = config_from_dict(tiny_raw("B"))
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (96, 6, 1, 32)
    assert cfg.head_dim * cfg.num_attention_heads != cfg.hidden_size
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and cfg.tie_word_embeddings is False
    spec = cfg.model_spec()
    assert len(spec.layers) == 3 and spec.vocab_size == 389
    assert spec.layers[0].mixer.scale == pytest.approx(32 ** -0.5)  # engine/model.py:130
    assert spec.layers[0].mixer.qk_norm.eps == 1e-5 and spec.layers[0].mixer.position.theta == 1e6


def test_head_dim_defaults_to_hidden_over_heads():
    raw = tiny_raw("A")
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == 64 // 4  # engine/model.py:47


def test_missing_keys_are_all_named():
    raw = tiny_raw("A")
    del raw["rms_norm_eps"], raw["rope_theta"], raw["vocab_size"]
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    for key in ("rms_norm_eps", "rope_theta", "vocab_size"):
        assert key in str(err.value)


def test_unknown_architecture_lists_known_ones():
    raw = tiny_raw("A")
    raw["architectures"] = ["SomethingElse"]
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(raw)
    assert "Qwen3ForCausalLM" in architecture_names()


@pytest.mark.parametrize("patch,word", [
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope scaling"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "head_dim"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
])
def test_options_that_are_not_built_are_refused(patch, word):
    raw = tiny_raw("A")
    raw.update(patch)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_windows_by_layer():
    cfg = config_from_dict(tiny_raw("W"))
    assert cfg.layer_windows == (None, 40, None, 40)
    raw = tiny_raw("A")
    raw.update(use_sliding_window=True, sliding_window=16, max_window_layers=1)
    assert config_from_dict(raw).layer_windows == (None, 16)
    assert [l.mixer.window for l in config_from_dict(raw).model_spec().layers] == [None, 16]


def test_round_trip_through_a_folder(tmp_path):
    for name in TINY:
        cfg = config_from_dict(tiny_raw(name))
        save_config(cfg, tmp_path / name)
        assert load_config(tmp_path / name) == cfg
        assert json.loads((tmp_path / name / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nowhere")
