"""Configuration and registry (no GPU)."""
import json
import os

import pytest

import helpers
from boring_llm_b200 import ConfigError, Qwen2Config, load_config, registered_architectures
from boring_llm_b200.config import EngineOptions, resolve_architecture


def base():
    return dict(helpers.TINY["A"])


def test_reads_every_size_from_its_key():
    c = Qwen2Config.from_dict(helpers.TINY["B"])
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 96, 3, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 200, 320)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert c.layer_windows == (0, 0, 0)


def test_head_dim_key_wins_over_division():
    c = Qwen2Config.from_dict(helpers.TINY["C"])
    assert c.head_dim == 48 and c.hidden_size // c.num_attention_heads == 16


def test_defaults_follow_the_reference():
    d = base()
    for k in ("num_key_value_heads", "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        d.pop(k)
    c = Qwen2Config.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads      # src/model.br:385
    assert c.rope_theta == 10000.0                             # src/model.br:393
    assert c.rms_norm_eps == 1e-6                              # src/model.br:398
    assert c.tie_word_embeddings is False


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads",
                                 "intermediate_size", "vocab_size"])
def test_missing_required_key(key):
    d = base()
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


def test_bad_values():
    for key, val, pat in [("num_attention_heads", 3, "multiple"), ("hidden_size", 0, "positive"),
                          ("vocab_size", "many", "int"), ("hidden_act", "gelu", "hidden_act"),
                          ("rms_norm_eps", 0.0, "rms_norm_eps"), ("num_hidden_layers", True, "integer")]:
        d = base()
        d[key] = val
        with pytest.raises(ConfigError, match=pat):
            Qwen2Config.from_dict(d)
    d = base()
    d["hidden_size"] = 66
    with pytest.raises(ConfigError, match="head_dim"):
        Qwen2Config.from_dict(d)
    d = base()
    d["head_dim"] = 15
    with pytest.raises(ConfigError, match="even"):
        Qwen2Config.from_dict(d)


def test_rope_scaling_is_refused_not_ignored():
    d = base()
    d["rope_scaling"] = {"type": "yarn", "factor": 4.0}
    with pytest.raises(ConfigError, match="rope_scaling"):
        Qwen2Config.from_dict(d)
    d["rope_scaling"] = None
    Qwen2Config.from_dict(d)


def test_windows():
    c = Qwen2Config.from_dict(helpers.TINY["C"])
    assert c.layer_windows == (0, 20, 20)
    d = dict(helpers.TINY["C"])
    d["layer_types"] = ["sliding_attention", "full_attention", "sliding_attention"]
    assert Qwen2Config.from_dict(d).layer_windows == (20, 0, 20)
    d["layer_types"] = ["full_attention"]
    with pytest.raises(ConfigError, match="layer_types"):
        Qwen2Config.from_dict(d)
    d = dict(helpers.TINY["C"])
    d["use_sliding_window"] = False
    assert Qwen2Config.from_dict(d).layer_windows == (0, 0, 0)
    d = dict(helpers.TINY["C"])
    d.pop("sliding_window")
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2Config.from_dict(d)


def test_round_trip_through_config_json(tmp_path):
    for name in helpers.TINY:
        c = Qwen2Config.from_dict(helpers.TINY[name])
        with open(tmp_path / "config.json", "w") as f:
            json.dump(c.to_dict(), f)
        assert load_config(str(tmp_path)) == c


def test_registry():
    assert "Qwen2ForCausalLM" in registered_architectures()
    assert resolve_architecture({"model_type": "qwen2"}).config_cls is Qwen2Config
    with pytest.raises(ConfigError, match="supported: .*Qwen2ForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve_architecture({})


def test_config_json_problems(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))


def test_engine_options():
    o = EngineOptions(dtype="bf16", max_num_batched_tokens=100, prefill_chunk=512)
    assert o.dtype == "bfloat16" and o.effective_prefill_chunk == 100     # src/cli_config.br:24-25
    assert EngineOptions(ctx_size=128, max_num_seqs=4).capacity_tokens == 512
    with pytest.raises(ValueError):
        EngineOptions(dtype="float16")
    with pytest.raises(ValueError):
        EngineOptions(page_size=0)
