"""Configuration and registry (CPU)."""
import json

import pytest

import tiny
from garlic_inference_b200 import ConfigError, Qwen3Config, load_config, register_architecture
from garlic_inference_b200.config import known_architectures
from garlic_inference_b200.engine import wanted_tensors


def _write(tmp_path, cfg: dict):
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    return tmp_path


def _full(name="A") -> dict:
    return tiny.make_config(name).to_dict()


def test_roundtrip_every_tiny_config(tmp_path):
    for name in tiny.TINY:
        d = tmp_path / name
        d.mkdir()
        cfg = load_config(_write(d, _full(name)))
        assert isinstance(cfg, Qwen3Config)
        assert cfg == tiny.make_config(name)


def test_no_size_stands_in_code():
    """Every size of the plan comes from the configuration: change one key, the plan follows."""
    base = tiny.TINY["B"]["cfg"]
    for key, new in [("hidden_size", 192), ("intermediate_size", 40), ("vocab_size", 123), ("head_dim", 64),
                     ("num_key_value_heads", 3), ("num_hidden_layers", 5)]:
        cfg = Qwen3Config(**{**base, key: new})
        wants = wanted_tensors(cfg.plan())
        h, d = cfg.hidden_size, cfg.head_dim
        assert wants["model.embed_tokens.weight"].shape == (cfg.vocab_size, h)
        assert wants["lm_head.weight"].shape == (cfg.vocab_size, h)
        assert wants["model.layers.0.self_attn.q_proj.weight"].shape == (cfg.num_attention_heads * d, h)
        assert wants["model.layers.0.self_attn.k_proj.weight"].shape == (cfg.num_key_value_heads * d, h)
        assert wants["model.layers.0.self_attn.o_proj.weight"].shape == (h, cfg.num_attention_heads * d)
        assert wants["model.layers.0.self_attn.q_norm.weight"].shape == (d,)
        assert wants["model.layers.0.mlp.down_proj.weight"].shape == (h, cfg.intermediate_size)
        assert f"model.layers.{cfg.num_hidden_layers - 1}.mlp.up_proj.weight" in wants
        assert f"model.layers.{cfg.num_hidden_layers}.mlp.up_proj.weight" not in wants


def test_tied_head_wants_no_lm_head():
    wants = wanted_tensors(tiny.make_config("A").plan())
    assert "lm_head.weight" not in wants
    plan = tiny.make_config("A").plan()
    assert plan.head.weights["weight"] == plan.embedding.weights["weight"]


def test_constants_reach_the_parts():
    cfg = tiny.make_config("C")
    plan = cfg.plan()
    assert [l.mixer.params["window"] for l in plan.layers] == [None, 40, 40, None]
    assert all(l.mixer.params["qk_norm_eps"] == 3e-5 for l in plan.layers)
    assert all(l.norms["input"].params["eps"] == 3e-5 for l in plan.layers)
    assert plan.positions["rotary"].params["theta"] == 5e5
    assert plan.final_norm.params["eps"] == 3e-5
    assert [(e.layer, e.cache, e.writes_cache) for e in plan.schedule] == [(i, i, True) for i in range(4)]


def test_window_from_max_window_layers():
    cfg = Qwen3Config(**{**tiny.TINY["B"]["cfg"], "sliding_window": 8, "use_sliding_window": True,
                         "max_window_layers": 1})
    assert cfg.layer_windows() == [None, 8, 8]
    off = Qwen3Config(**{**tiny.TINY["B"]["cfg"], "sliding_window": 8, "use_sliding_window": False})
    assert off.layer_windows() == [None, None, None]


def test_head_dim_defaults_to_hidden_over_heads(tmp_path):
    cfg = _full("A")
    del cfg["head_dim"]
    assert load_config(_write(tmp_path, cfg)).head_dim == 16


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "intermediate_size", "vocab_size",
                                 "max_position_embeddings"])
def test_missing_key_is_named(tmp_path, key):
    cfg = _full()
    del cfg[key]
    with pytest.raises(ConfigError, match=key):
        load_config(_write(tmp_path, cfg))


@pytest.mark.parametrize("patch,word", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": "64"}, "integer"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "sliding_attention"], "sliding_window": None}, "sliding_window"),
])
def test_refused_options_are_named(tmp_path, patch, word):
    with pytest.raises(ConfigError, match=word):
        load_config(_write(tmp_path, {**_full(), **patch}))


def test_unknown_architecture_lists_known(tmp_path):
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        load_config(_write(tmp_path, {**_full(), "architectures": ["LlamaForCausalLM"]}))
    with pytest.raises(ConfigError, match="architectures"):
        load_config(_write(tmp_path, {k: v for k, v in _full().items() if k != "architectures"}))
    with pytest.raises(ConfigError, match="config.json"):
        load_config(tmp_path / "nowhere")


def test_registering_another_architecture(tmp_path):
    class ToyConfig(Qwen3Config):
        pass

    register_architecture("ToyForCausalLM", ToyConfig)
    assert "ToyForCausalLM" in known_architectures()
    cfg = load_config(_write(tmp_path, {**_full(), "architectures": ["ToyForCausalLM"]}))
    assert type(cfg) is ToyConfig
    with pytest.raises(TypeError):
        register_architecture("Broken", object)
