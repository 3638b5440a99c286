"""Configuration, registry and the model description built from them (no GPU)."""
import copy

import pytest

import tiny
from spissa_b200.config import (ConfigError, LlamaConfig, ModelSpec, PartSpec, ScheduleEntry, UnknownArchitecture,
                                config_from_dict, known_architectures, load_config, register_architecture,
                                unregister_architecture)
from spissa_b200.engine.model import Model


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_tiny_configs_parse_and_round_trip(name):
    d = tiny.TINIES[name][0]
    cfg = config_from_dict(d)
    assert isinstance(cfg, LlamaConfig)
    assert cfg.hidden_size == d["hidden_size"] and cfg.head_dim == d["head_dim"]
    assert cfg.num_key_value_heads == d["num_key_value_heads"]
    again = config_from_dict(cfg.to_dict())
    assert again == cfg


def test_defaults_follow_the_reference():
    d = dict(architectures=["LlamaForCausalLM"], vocab_size=10, hidden_size=8, intermediate_size=16,
             num_hidden_layers=1, num_attention_heads=2)
    cfg = config_from_dict(d)
    assert cfg.num_key_value_heads == 2 and cfg.head_dim == 4
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0 and cfg.max_position_embeddings == 2048
    assert cfg.rope_scaling is None and cfg.tie_word_embeddings is False


@pytest.mark.parametrize("drop", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                  "num_attention_heads"])
def test_missing_required_field_is_named(drop):
    d = copy.deepcopy(tiny.TINY_A)
    del d[drop]
    with pytest.raises(ConfigError, match=drop):
        config_from_dict(d)


def test_bad_shapes_are_refused():
    d = copy.deepcopy(tiny.TINY_A)
    d["num_key_value_heads"] = 3
    with pytest.raises(ConfigError, match="multiple"):
        config_from_dict(d)
    d = copy.deepcopy(tiny.TINY_A)
    d["head_dim"] = 15
    with pytest.raises(ConfigError, match="even"):
        config_from_dict(d)
    d = copy.deepcopy(tiny.TINY_A)
    del d["head_dim"]
    d["hidden_size"] = 66
    with pytest.raises(ConfigError, match="divisible"):
        config_from_dict(d)
    d = copy.deepcopy(tiny.TINY_A)
    d["num_hidden_layers"] = 0
    with pytest.raises(ConfigError, match="positive"):
        config_from_dict(d)
    d = copy.deepcopy(tiny.TINY_A)
    d["attention_bias"] = True
    with pytest.raises(ConfigError, match="attention_bias"):
        config_from_dict(d)


def test_rope_scaling_kinds():
    d = copy.deepcopy(tiny.TINY_B)
    assert config_from_dict(d).rope_scaling.rope_type == "llama3"
    d["rope_scaling"] = {"rope_type": "yarn", "factor": 2.0}
    with pytest.raises(ConfigError, match="yarn"):
        config_from_dict(d)
    d["rope_scaling"] = {"rope_type": "llama3", "factor": 2.0}
    with pytest.raises(ConfigError, match="low_freq_factor"):
        config_from_dict(d)
    d["rope_scaling"] = {"type": "linear", "factor": 4.0}
    assert config_from_dict(d).rope_scaling.factor == 4.0


def test_unknown_architecture_lists_known_names():
    with pytest.raises(UnknownArchitecture, match="LlamaForCausalLM"):
        config_from_dict(dict(architectures=["NopeForCausalLM"]))
    assert "LlamaForCausalLM" in known_architectures()
    # model_type alone is enough, as in the reference's normaliser
    d = copy.deepcopy(tiny.TINY_A)
    del d["architectures"]
    assert isinstance(config_from_dict(d), LlamaConfig)


def test_load_config_from_folder(tmp_path):
    import json
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_B))
    assert load_config(tmp_path).vocab_size == 384
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nothing")


def test_spec_names_every_part_and_no_size_is_hidden():
    cfg = config_from_dict(tiny.TINY_B)
    spec = cfg.to_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    att = spec.layers[1].mixer
    assert att.kind == "attention" and att.params["num_kv_heads"] == 1 and att.params["head_dim"] == 32
    assert att.params["position"].params["scaling"]["rope_type"] == "llama3"
    assert spec.layers[1].norms["ffn"].params["eps"] == 1e-6
    assert spec.head.params["tied_to"] is None
    assert config_from_dict(tiny.TINY_A).to_spec().head.params["tied_to"] == "model.embed_tokens.weight"


def test_model_lists_the_checkpoint_names():
    m = Model(config_from_dict(tiny.TINY_A).to_spec())
    names = {s.name: s.shape for s in m.weight_specs()}
    assert names["model.embed_tokens.weight"] == (256, 64)
    assert names["model.layers.1.self_attn.k_proj.weight"] == (32, 64)
    assert names["model.layers.0.mlp.down_proj.weight"] == (64, 192)
    assert names["model.norm.weight"] == (64,)
    assert "lm_head.weight" not in names
    assert len(names) == 1 + 2 * 9 + 1
    mb = Model(config_from_dict(tiny.TINY_B).to_spec())
    assert "lm_head.weight" in {s.name for s in mb.weight_specs()}


def test_schedule_is_data_and_is_checked():
    spec = config_from_dict(tiny.TINY_A).to_spec()
    twice = ModelSpec(**{**spec.__dict__, "schedule": (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
                                                       ScheduleEntry(1, 1, writes_cache=False))})
    twice.validate()
    m = Model(twice)
    assert sorted(m.cache_requests()) == [0, 1, 2]
    bad = ModelSpec(**{**spec.__dict__, "schedule": (ScheduleEntry(0, 0), ScheduleEntry(1, 0))})
    with pytest.raises(ValueError, match="both write"):
        bad.validate()
    bad = ModelSpec(**{**spec.__dict__, "schedule": (ScheduleEntry(0, 5, writes_cache=False),)})
    with pytest.raises(ValueError, match="before any entry writes"):
        bad.validate()
    bad = ModelSpec(**{**spec.__dict__, "schedule": (ScheduleEntry(7, 0),)})
    with pytest.raises(ValueError, match="names layer 7"):
        bad.validate()


def test_another_architecture_registers_without_touching_the_library():
    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d)

        def to_spec(self):
            return config_from_dict({**tiny.TINY_A, "num_hidden_layers": self.d["depth"]}).to_spec()

    register_architecture("ToyForCausalLM", ToyConfig)
    try:
        cfg = config_from_dict(dict(architectures=["ToyForCausalLM"], depth=1))
        assert len(cfg.to_spec().layers) == 1
    finally:
        unregister_architecture("ToyForCausalLM")
    with pytest.raises(UnknownArchitecture):
        config_from_dict(dict(architectures=["ToyForCausalLM"], depth=1))
