"""Configuration gate, architecture registry and engine knobs (no GPU)."""
import json

import pytest

from tiny_configs import TINY_A, TINY_B
import tessweave_engine_b200 as tw
from tessweave_engine_b200.config import ConfigError, EngineConfig, Qwen2Config, architectures, resolve, resolve_folder


def test_fields_and_defaults():
    cfg = Qwen2Config.from_dict(TINY_A)
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (64, 4, 2, 16)
    assert cfg.tie_word_embeddings and cfg.eos_token_ids == (255,)
    minimal = {"model_type": "qwen2", "vocab_size": 10, "hidden_size": 32, "intermediate_size": 8,
               "num_hidden_layers": 1, "num_attention_heads": 4, "max_position_embeddings": 64}
    d = Qwen2Config.from_dict(minimal)
    # defaults of flow_engine/config.py:38-48
    assert d.num_key_value_heads == 4 and d.head_dim == 8 and d.rms_norm_eps == 1e-6 and d.rope_theta == 10000.0
    assert d.tie_word_embeddings is False and d.eos_token_ids == ()


@pytest.mark.parametrize("change", [
    {"model_type": "llama"}, {"model_type": "mistral"}, {"use_sliding_window": True},
    {"rope_scaling": {"rope_type": "yarn", "factor": 4}}, {"quantization_config": {"bits": 4}},
    {"auto_map": {"AutoModel": "x.Y"}}, {"hidden_act": "gelu"}, {"mlp_bias": True}, {"num_experts": 8},
    {"num_local_experts": 4}, {"num_key_value_heads": 3}, {"head_dim": 15}, {"hidden_size": 65},
    {"vocab_size": 0}, {"num_hidden_layers": 0}, {"rms_norm_eps": 0.0},
])
def test_unsupported_semantics_are_refused_before_weights(change):
    with pytest.raises(ConfigError):
        Qwen2Config.from_dict({**TINY_A, **change})


def test_default_rope_scaling_is_accepted():
    Qwen2Config.from_dict({**TINY_A, "rope_scaling": {"rope_type": "default"}})
    Qwen2Config.from_dict({**TINY_A, "rope_scaling": None})


def test_missing_required_key():
    broken = dict(TINY_A)
    del broken["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        Qwen2Config.from_dict(broken)


def test_registry_builds_spec_from_config_only():
    assert "Qwen2ForCausalLM" in architectures()
    for config in (TINY_A, TINY_B):
        cfg, spec = resolve(config)
        assert len(spec.layers) == len(spec.schedule) == config["num_hidden_layers"]
        mixer = spec.layers[0].block.params["mixer"].params
        assert mixer["n_heads"] == config["num_attention_heads"] and mixer["head_dim"] == config["head_dim"]
        assert mixer["position"].params["theta"] == config["rope_theta"]
        assert spec.layers[0].block.params["norm1"].params["eps"] == config["rms_norm_eps"]
        assert spec.tie_word_embeddings == config["tie_word_embeddings"]
    with pytest.raises(ConfigError, match="not registered"):
        resolve({**TINY_A, "architectures": ["SomethingElseForCausalLM"]})
    no_arch = {k: v for k, v in TINY_A.items() if k != "architectures"}
    assert resolve(no_arch)[0].architecture == "Qwen2ForCausalLM"      # found through model_type


def test_generation_config_overrides_eos(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 4], "temperature": 0.7}))
    cfg, _ = resolve_folder(tmp_path)
    assert cfg.eos_token_ids == (3, 4)


def test_engine_config_validation():
    EngineConfig()
    for bad in ({"block_size": 0}, {"kv_blocks": -1}, {"max_active": 0}, {"prefill_chunk": 4, "min_prefill_chunk": 8},
                {"target_step_ms": 0}, {"max_step_tokens": 1}):
        with pytest.raises(ValueError):
            EngineConfig(**bad)
    assert EngineConfig(max_active=4, prefill_chunk=32).step_token_budget == 36
    assert EngineConfig(max_step_tokens=10).step_token_budget == 10
