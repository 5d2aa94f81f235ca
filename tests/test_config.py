"""Configuration: the architecture's own config.json keys, defaults, refusals,
the registry, and the lowering to a model specification."""
import json

import pytest

from tiny_configs import TINY, TINY_A, TINY_B, TINY_C
from zlm_b200 import ConfigError, Qwen3Config
from zlm_b200.registry import ARCHITECTURES, config_from_dict, config_from_folder


def test_registry_maps_the_architecture_name():
    assert ARCHITECTURES["Qwen3ForCausalLM"] is Qwen3Config
    cfg = config_from_dict(TINY_B)
    assert isinstance(cfg, Qwen3Config)
    with pytest.raises(ConfigError, match="unsupported architecture 'LlamaForCausalLM'.*Qwen3ForCausalLM"):
        config_from_dict({**TINY_A, "architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_every_size_comes_from_the_keys():
    a, b, c = (config_from_dict(TINY[n]) for n in "ABC")
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size, a.rope_theta, a.rms_norm_eps, a.tie_word_embeddings,
            a.max_position_embeddings) == (2, 64, 4, 2, 16, 128, 256, 10000.0, 1e-6, True, 128)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim,
            b.intermediate_size, b.vocab_size, b.rope_theta, b.rms_norm_eps, b.tie_word_embeddings,
            b.max_position_embeddings) == (3, 96, 6, 3, 32, 160, 320, 1e6, 1e-5, False, 256)
    assert b.num_attention_heads * b.head_dim != b.hidden_size
    assert c.layer_windows == (0, 24, 0, 24)


def test_defaults_follow_the_reference():
    d = {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
         "num_attention_heads": 4, "intermediate_size": 128, "vocab_size": 100, "max_position_embeddings": 64}
    cfg = config_from_dict(d)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 16
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 1_000_000.0 and not cfg.tie_word_embeddings
    assert config_from_dict({**d, "rope_theta": 500000}).rope_theta == 500000.0     # integer accepted


@pytest.mark.parametrize("patch,match", [
    ({"hidden_size": None}, "missing key 'hidden_size'"),
    ({"num_hidden_layers": "two"}, "'num_hidden_layers' must be an integer"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"head_dim": 15}, "head_dim=15 must be even"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act='gelu'"),
    ({"num_experts": 8}, "mixture-of-experts"),
    ({"layer_types": ["full_attention"]}, "'layer_types' must list 2 layers"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "sliding_window"),
    ({"use_sliding_window": True}, "positive 'sliding_window'"),
    ({"tie_word_embeddings": "yes"}, "true or false"),
])
def test_refusals_name_the_key(patch, match):
    with pytest.raises(ConfigError, match=match):
        config_from_dict({**TINY_A, **patch})


def test_windows_from_the_keys():
    base = {**TINY_B}
    assert config_from_dict(base).layer_windows == (0, 0, 0)
    w = config_from_dict({**base, "use_sliding_window": True, "sliding_window": 32, "max_window_layers": 1})
    assert w.layer_windows == (0, 32, 32)
    # a window that is set but not switched on is not used
    assert config_from_dict({**base, "sliding_window": 32}).layer_windows == (0, 0, 0)


def test_round_trip_through_a_folder(tmp_path):
    cfg = config_from_dict(TINY_C)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert config_from_folder(str(tmp_path)) == cfg
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_folder(str(tmp_path / "nowhere"))


def test_model_spec_is_data():
    spec = config_from_dict(TINY_C).to_model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and all(e.cache_of is None for e in spec.schedule)
    assert [l.mixer.params["window"] for l in spec.layers] == [0, 24, 0, 24]
    assert spec.layers[1].mixer.kind == "gqa_attention" and spec.layers[1].feed_forward.kind == "swiglu"
    assert spec.layers[2].mixer.tensor_name("q_proj.weight") == "model.layers.2.self_attn.q_proj.weight"
    assert spec.layers[0].mixer.params["position"]["theta"] == 50000.0


def test_schedule_validation():
    from dataclasses import replace
    from zlm_b200.config import ScheduleEntry
    spec = config_from_dict(TINY_A).to_model_spec()
    replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))).validate()
    with pytest.raises(ConfigError, match="names layer 5"):
        replace(spec, schedule=(ScheduleEntry(5),)).validate()
    with pytest.raises(ConfigError, match="earlier entry"):
        replace(spec, schedule=(ScheduleEntry(0, cache_of=1), ScheduleEntry(1))).validate()


def test_rope_parameters_object_is_read_and_what_it_may_hide_is_refused():
    """A config.json from a newer writer carries the rotary base inside ``rope_parameters``
    and no top-level ``rope_theta``: the base must come from there, not from the default."""
    base = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    moved = {**base, "rope_parameters": {"rope_theta": 10000.0, "rope_type": "default"}}
    assert config_from_dict(moved).rope_theta == 10000.0
    assert config_from_dict({**moved, "rope_theta": 10000}).rope_theta == 10000.0
    assert config_from_dict({**base, "rope_parameters": {"rope_type": "default"}}).rope_theta == 1_000_000.0
    assert config_from_dict({**TINY_A, "rope_parameters": {"rope_type": "default"}}).rope_theta == 10000.0
    assert config_from_dict({**TINY_A, "rope_scaling": {"rope_type": "default"}}).rope_theta == 10000.0
    with pytest.raises(ConfigError, match="differ"):
        config_from_dict({**moved, "rope_theta": 1e6})
    for bad in ({"rope_theta": 1e4, "rope_type": "yarn", "factor": 4.0},
                {"rope_theta": 1e4, "rope_type": "linear"},
                {"rope_theta": 1e4, "rope_type": "default", "factor": 2.0},
                {"rope_theta": 1e4, "partial_rotary_factor": 0.5},
                {"rope_theta": 1e4, "mrope_section": [1, 2]}):
        with pytest.raises(ConfigError, match="rope_parameters"):
            config_from_dict({**base, "rope_parameters": bad})
    with pytest.raises(ConfigError, match="partial_rotary_factor"):
        config_from_dict({**TINY_A, "partial_rotary_factor": 0.5})
    with pytest.raises(ConfigError, match="must be an object"):
        config_from_dict({**base, "rope_parameters": 3})
