"""Configuration and registry (no GPU)."""
import json
import os

import pytest

from gophonic_b200 import registry
from gophonic_b200.config import ConfigError, Qwen3Config

BASE = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 96, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 256,
    "vocab_size": 1000, "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "rope_theta": 1e6,
    "rope_scaling": None, "attention_bias": False, "hidden_act": "silu", "tie_word_embeddings": False,
}


def test_reads_every_key():
    c = Qwen3Config.from_dict(BASE)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (96, 3, 6, 3)
    assert (c.head_dim, c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (32, 256, 1000, 1024)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and not c.tie_word_embeddings
    assert c.q_dim == 192 and c.kv_dim == 96


def test_head_dim_defaults_to_hidden_over_heads():
    d = dict(BASE)
    del d["head_dim"]
    assert Qwen3Config.from_dict(d).head_dim == 16
    d["head_dim"] = 0
    assert Qwen3Config.from_dict(d).head_dim == 16


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "vocab_size", "max_position_embeddings", "rms_norm_eps",
                                 "rope_theta"])
def test_missing_key_is_named(key):
    d = dict(BASE)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"model_type": "llama"}, "model_type"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"attention_bias": True}, "attention_bias"),
    ({"use_sliding_window": True}, "use_sliding_window"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_attention_heads": 7}, "num_attention_heads"),
    ({"head_dim": 31}, "head_dim"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"rope_theta": -1}, "rope_theta"),
    ({"hidden_size": 0}, "hidden_size"),
    ({"vocab_size": (16 << 20) + 1}, "vocab_size"),
    ({"num_hidden_layers": "3"}, "num_hidden_layers"),
])
def test_rejected_variants(patch, word):
    d = dict(BASE)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(d)


def test_round_trip_through_json(tmp_path):
    c = Qwen3Config.from_dict(BASE)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(c.to_dict(), f)
    assert registry.read_config(str(tmp_path)) == c
    assert Qwen3Config.from_json(str(tmp_path)) == c


def test_registry_selects_by_architecture_then_model_type(tmp_path):
    assert registry.architecture_of(BASE) == "Qwen3ForCausalLM"
    assert registry.architecture_of({"model_type": "qwen3"}) == "Qwen3ForCausalLM"
    with pytest.raises(registry.RegistryError, match="Qwen3ForCausalLM"):
        registry.architecture_of({"architectures": ["NoSuchModel"], "model_type": "nope"})


def test_model_spec_is_data():
    c = Qwen3Config.from_dict(BASE)
    spec = c.model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert (m.kind, m.heads, m.kv_heads, m.head_dim, m.window) == ("attention", 6, 3, 32, 0)
    assert m.qk_norm.eps == 1e-5 and m.position.theta == 1e6 and m.position.rotary_dim == 32
    assert abs(m.scale - 32 ** -0.5) < 1e-15
    assert spec.layers[1].feed_forward.intermediate == 256
    assert spec.head.tied_to == "model.embed_tokens.weight"


def test_schedule_validation():
    from dataclasses import replace
    from gophonic_b200.config import ScheduleEntry
    spec = Qwen3Config.from_dict(BASE).model_spec()
    replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(2, cache_of=1))).validate()
    with pytest.raises(ValueError, match="names layer 5"):
        replace(spec, schedule=(ScheduleEntry(5),)).validate()
    with pytest.raises(ValueError, match="does not run before"):
        replace(spec, schedule=(ScheduleEntry(0, cache_of=0),)).validate()
    with pytest.raises(ValueError, match="no cache of its own"):
        replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(2, cache_of=1))).validate()


def test_part_registry_errors_and_replacement():
    from gophonic_b200 import parts  # registers built-ins
    assert registry.part_class("mixer", "attention") is parts.Attention
    with pytest.raises(registry.RegistryError, match="no mixer part of kind 'conv'"):
        registry.part_class("mixer", "conv")

    class Dummy:
        pass
    registry.register_mixer("dummy-for-test", Dummy)
    assert registry.part_class("mixer", "dummy-for-test") is Dummy


def test_stop_ids_come_from_the_model_folder(tmp_path):
    import json
    from gophonic_b200.api import read_stop_ids
    d = tmp_path / "m"
    d.mkdir()
    assert read_stop_ids(str(d)) == []
    (d / "config.json").write_text(json.dumps({"eos_token_id": 7}))
    assert read_stop_ids(str(d)) == [7]
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": [151645, 151643]}))
    assert read_stop_ids(str(d)) == [151645, 151643]          # the generation config wins
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": "x"}))
    assert read_stop_ids(str(d)) == [7]                         # what is no id or list of ids is passed over


def test_named_configurations_are_config_files_read_like_any_other():
    from gophonic_b200 import registry
    from gophonic_b200.api import ErrUnknownFormat, _parse_random, random_model_path
    from gophonic_b200.config.presets import preset, preset_names
    assert preset_names() == ["1.7b", "32b", "8b", "tinyA", "tinyB"]
    for name in preset_names():
        raw = preset(name)
        cfg = registry.config_class(registry.architecture_of(raw)).from_dict(raw)
        assert cfg.to_dict()["hidden_size"] == raw["hidden_size"]
    big = preset("8b")
    assert (big["num_hidden_layers"], big["hidden_size"], big["intermediate_size"], big["vocab_size"]) == (36, 4096, 12288, 151936)
    cfg, seed = _parse_random(random_model_path("8b", seed=5, layers=2))
    assert seed == 5 and cfg.num_hidden_layers == 2 and cfg.hidden_size == 4096
    assert _parse_random("random:tinyB")[0].vocab_size == 1000
    with pytest.raises(ErrUnknownFormat, match="no configuration named"):
        _parse_random("random:70b")
    with pytest.raises(ValueError, match="layers=99"):
        _parse_random("random:8b?layers=99")
    with pytest.raises(ValueError, match="unknown option"):
        _parse_random("random:8b?depth=2")


def test_command_line_refuses_what_it_cannot_run(tmp_path, capsys):
    from gophonic_b200.__main__ import main
    assert main([]) == 2
    assert main(["-model", "x", "-random-config", "tinyA", "1"]) == 2
    assert main(["-random-config", "tinyA"]) == 1 and "no prompt" in capsys.readouterr().err
    assert main(["-model", "x", "1,b"]) == 2
    assert main(["-model", str(tmp_path), "-write-model", str(tmp_path / "out"), "1"]) == 1
    out = tmp_path / "written"
    assert main(["-random-config", "tinyB", "-weights-seed", "9", "-layers", "1", "-write-model", str(out)]) == 0
    from gophonic_b200.config import Qwen3Config
    assert Qwen3Config.from_json(str(out)).num_hidden_layers == 1 and (out / "model.safetensors").exists()
