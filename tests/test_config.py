"""Configuration: keys of config.json, defaults, validation, registry."""
import json

import pytest

from tiny_configs import TINY_A, TINY_B
from nanoinfer_b200.config import ConfigError, config_from_dict, load_config, registered_architectures
from nanoinfer_b200.config.model_config import LayerRun, ModelConfig


def test_tiny_b_fields():
    cfg = config_from_dict(TINY_B)
    assert cfg.architecture == "LlamaForCausalLM" and cfg.hidden_size == 96 and cfg.vocab_size == 384
    assert cfg.num_layers == 3 and [r.layer for r in cfg.schedule] == [0, 1, 2]
    m = cfg.layers[0].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.window) == (3, 1, 32, None)
    assert m.softmax_scale == pytest.approx(32 ** -0.5)
    assert m.position.theta == 500000.0 and m.position.scaling.factor == 32.0
    assert m.position.scaling.original_max_position_embeddings == 64 and m.position.pairing == "half"
    assert cfg.layers[0].feed_forward.intermediate_size == 256
    assert cfg.layers[0].mixer_norm.eps == 1e-6 and cfg.final_norm.eps == 1e-6
    assert cfg.tie_word_embeddings is False and cfg.eos_token_ids == (2, 3)


def test_defaults_follow_the_reference():
    raw = {"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 128,
           "num_hidden_layers": 1, "num_attention_heads": 4, "vocab_size": 50, "max_position_embeddings": 32}
    cfg = config_from_dict(raw)
    m = cfg.layers[0].mixer
    assert m.num_kv_heads == 4 and m.head_dim == 16          # MHA and dim / heads
    assert cfg.final_norm.eps == 1e-5 and m.position.theta == 10000.0 and m.position.scaling is None
    assert cfg.tie_word_embeddings is False and cfg.eos_token_ids == () and cfg.bos_token_id is None


@pytest.mark.parametrize("change,msg", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_attention_heads": 5}, "multiple"),
    ({"head_dim": None, "hidden_size": 66}, "head_dim"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"architectures": ["NoSuchModel"]}, "LlamaForCausalLM"),
    ({"architectures": []}, "architectures"),
    ({"rope_pairing": "odd"}, "rope_pairing"),
    ({"eos_token_id": "x"}, "eos_token_id"),
])
def test_bad_configs_are_refused(change, msg):
    raw = dict(TINY_A)
    for k, v in change.items():
        if v is None:
            raw.pop(k, None)
        else:
            raw[k] = v
    with pytest.raises(ConfigError, match=msg):
        config_from_dict(raw)


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert load_config(str(tmp_path)).hidden_size == 64
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))


def test_registry_lists_llama():
    assert "LlamaForCausalLM" in registered_architectures()


def test_schedule_validation():
    cfg = config_from_dict(TINY_A)

    def with_schedule(s):
        return ModelConfig(**{**cfg.__dict__, "schedule": tuple(s)})

    with_schedule([LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(1, cache_of=1)]).validate()
    with pytest.raises(ConfigError, match="names layer"):
        with_schedule([LayerRun(2)]).validate()
    with pytest.raises(ConfigError, match="earlier run"):
        with_schedule([LayerRun(0, cache_of=0)]).validate()
    with pytest.raises(ConfigError, match="no cache of its own"):
        with_schedule([LayerRun(0), LayerRun(1, cache_of=0), LayerRun(1, cache_of=1)]).validate()


def test_presets_are_configurations_of_the_family():
    """The package's config.json files of the published sizes parse like any other; the command
    line's random-model takes one of them or a file, not both and not neither."""
    from nanoinfer_b200.config import preset, preset_names
    assert preset_names() == ["llama-3.1-8b", "llama-3.2-1b", "llama-3.2-3b"]
    sizes = {}
    for name in preset_names():
        cfg = config_from_dict(preset(name))
        m = cfg.layers[0].mixer
        sizes[name] = (cfg.num_layers, cfg.hidden_size, m.num_heads, m.num_kv_heads, m.head_dim,
                       cfg.layers[0].feed_forward.intermediate_size, cfg.tie_word_embeddings)
        assert cfg.vocab_size == 128256 and m.position.theta == 500000.0 and cfg.final_norm.eps == 1e-5
    assert sizes["llama-3.2-1b"] == (16, 2048, 32, 8, 64, 8192, True)
    assert sizes["llama-3.2-3b"] == (28, 3072, 24, 8, 128, 8192, True)
    assert sizes["llama-3.1-8b"] == (32, 4096, 32, 8, 128, 14336, False)
    assert config_from_dict(preset("llama-3.1-8b")).layers[0].mixer.position.scaling.factor == 8.0
    with pytest.raises(KeyError, match="llama-3.2-1b"):
        preset("llama-9")
    from nanoinfer_b200.cli import main
    assert main(["random-model", "--out", "unused"]) == 2
    assert main(["random-model", "--out", "unused", "--preset", "llama-3.2-1b", "--config", "x.json"]) == 2
