"""Configuration and registry (no GPU)."""
import copy
import json
import os
import tempfile

import pytest

from agave_b200.config import (ConfigError, Gemma3Config, load_config, registered_architectures,
                               resolve_architecture)
import agave_b200  # noqa: F401  (registers architectures)
from util import TINY_A, TINY_B


def test_registry_resolves_by_architecture_and_model_type():
    assert "Gemma3ForCausalLM" in registered_architectures()
    assert resolve_architecture(TINY_A).name == "Gemma3ForCausalLM"
    assert resolve_architecture({"model_type": "gemma3_text"}).name == "Gemma3ForCausalLM"
    assert resolve_architecture({"model_type": "gemma3",
                                 "text_config": {"model_type": "gemma3_text"}}).name \
        == "Gemma3ForCausalLM"
    with pytest.raises(ConfigError) as e:
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    assert "Gemma3ForCausalLM" in str(e.value)


def test_sizes_come_from_the_file():
    a, b = Gemma3Config.from_dict(TINY_A), Gemma3Config.from_dict(TINY_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 1, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 6, 2, 32)
    assert a.rope_scaling_factor == 1.0 and b.rope_scaling_factor == 2.0
    assert a.eos_token_ids == (1,) and b.eos_token_ids == (1, 106)
    assert b.rms_norm_eps == 1e-5 and b.query_pre_attn_scalar == 24


def test_layer_pattern_and_list():
    a = Gemma3Config.from_dict(TINY_A)
    assert [a.is_local(l) for l in range(4)] == [True, False, True, False]
    b = Gemma3Config.from_dict(TINY_B)
    assert [b.is_local(l) for l in range(7)] == [True, True, False, True, True, False, True]
    d = dict(TINY_A)
    d["layer_types"] = ["full_attention", "sliding_attention", "sliding_attention",
                        "full_attention"]
    c = Gemma3Config.from_dict(d)
    assert [c.is_local(l) for l in range(4)] == [False, True, True, False]
    d["layer_types"] = ["full_attention"]
    with pytest.raises(ConfigError):
        Gemma3Config.from_dict(d)


def test_spec_carries_per_layer_parts():
    spec = Gemma3Config.from_dict(TINY_B).to_model_spec()
    assert len(spec.blocks) == 7 and [c.block for c in spec.schedule] == list(range(7))
    local, glob = spec.blocks[0].mixer, spec.blocks[2].mixer
    assert local.window == 16 and glob.window is None
    assert local.position.theta == 5000.0 and local.position.factor == 1.0
    assert glob.position.theta == 500000.0 and glob.position.factor == 2.0
    assert abs(local.scale - 24 ** -0.5) < 1e-12
    assert abs(spec.embed_scale - 96 ** 0.5) < 1e-12
    assert spec.blocks[0].norm.eps == 1e-5 and spec.blocks[0].norm.zero_centered


def test_text_config_overrides_and_rope_parameters():
    d = {"architectures": ["Gemma3ForConditionalGeneration"], "model_type": "gemma3",
         "text_config": dict(TINY_A)}
    c = Gemma3Config.from_dict(d)
    assert c.hidden_size == 64
    d2 = dict(TINY_A)
    d2.pop("rope_theta"); d2.pop("rope_local_base_freq"); d2.pop("rope_scaling")
    d2["rope_parameters"] = {
        "full_attention": {"rope_type": "linear", "factor": 8.0, "rope_theta": 1e6},
        "sliding_attention": {"rope_type": "default", "rope_theta": 1e4}}
    c2 = Gemma3Config.from_dict(d2)
    assert c2.rope_scaling_factor == 8.0 and c2.rope_theta == 1e6


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "head_dim", "vocab_size",
                                 "intermediate_size", "num_attention_heads"])
def test_missing_size_is_an_error_that_names_the_key(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError) as e:
        Gemma3Config.from_dict(d)
    assert key in str(e.value)


def test_bad_values():
    for key, val in [("num_key_value_heads", 3), ("head_dim", 15), ("rms_norm_eps", 0),
                     ("final_logit_softcapping", 30.0), ("attention_bias", True),
                     ("hidden_activation", "relu")]:
        d = dict(TINY_A)
        d[key] = val
        with pytest.raises(ConfigError):
            Gemma3Config.from_dict(d)
    d = dict(TINY_A)
    d["sliding_window"] = None
    with pytest.raises(ConfigError):
        Gemma3Config.from_dict(d)
    d = dict(TINY_A)
    d["rope_scaling"] = {"rope_type": "yarn", "factor": 2.0}
    with pytest.raises(ConfigError):
        Gemma3Config.from_dict(d)


def test_round_trip_through_config_json():
    c = Gemma3Config.from_dict(TINY_B)
    d = tempfile.mkdtemp()
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(c.to_dict(), f)
    entry, c2 = load_config(d)
    assert entry.name == "Gemma3ForCausalLM" and c2 == c
