"""Typed view of a Qwen2 ``config.json``.

Every size and constant of the model comes from here; nothing downstream
hard-codes one.  The gate mirrors the reference's ``ModelConfig.from_dict``
(flow_engine/config.py:23-52): anything whose semantics this engine does not
implement is refused *before* a single weight is read, rather than silently
approximated.  Unlike the reference, ``model_type == "llama"`` is refused too:
this engine carries one architecture.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, replace
from pathlib import Path


class ConfigError(ValueError):
    """config.json asks for something this engine does not implement."""


def _eos_tuple(value) -> tuple[int, ...]:
    if value is None:
        return ()
    if isinstance(value, int):
        return (int(value),)
    return tuple(int(v) for v in value)


@dataclass(frozen=True)
class Qwen2Config:
    """Fields follow the config.json keys of ``Qwen2ForCausalLM``.

    Defaults are those of flow_engine/config.py:38-48: ``num_key_value_heads``
    falls back to ``num_attention_heads``, ``head_dim`` to
    ``hidden_size // num_attention_heads``, ``rms_norm_eps`` to 1e-6,
    ``rope_theta`` to 10000, ``tie_word_embeddings`` to False.
    """

    architecture: str
    model_type: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...] = ()
    initializer_range: float = 0.02

    # ---- construction -------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen2Config":
        if d.get("model_type") != "qwen2":
            raise ConfigError(
                f"model_type {d.get('model_type')!r} is not supported: this engine runs the dense "
                "qwen2 decoder with full attention and default RoPE only")
        if d.get("quantization_config"):
            raise ConfigError("quantized checkpoints are not supported by the dense loader")
        scaling = d.get("rope_scaling")
        if scaling and scaling.get("rope_type", scaling.get("type")) != "default":
            raise ConfigError("scaled RoPE needs its own implementation; refusing a silent approximation")
        if d.get("use_sliding_window"):
            raise ConfigError("use_sliding_window=true is not implemented for qwen2")
        if d.get("hidden_act", "silu") != "silu" or d.get("mlp_bias"):
            raise ConfigError("only the unbiased SwiGLU feed-forward (hidden_act=silu) is supported")
        if d.get("num_local_experts") or d.get("num_experts") or d.get("auto_map"):
            raise ConfigError("expert models and checkpoints that need remote code are not supported")
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "max_position_embeddings"):
            if key not in d:
                raise ConfigError(f"config.json lacks the required key {key!r}")
        hidden = int(d["hidden_size"])
        heads = int(d["num_attention_heads"])
        if heads <= 0:
            raise ConfigError("num_attention_heads must be positive")
        kv_heads = int(d.get("num_key_value_heads") or heads)
        head_dim = int(d.get("head_dim") or hidden // heads)
        if min(hidden, kv_heads, head_dim) <= 0 or heads % kv_heads or hidden != heads * head_dim or head_dim % 2:
            raise ConfigError(
                "invalid attention sizes: need num_attention_heads % num_key_value_heads == 0, "
                "hidden_size == num_attention_heads * head_dim and an even head_dim")
        arch = d.get("architectures") or ["Qwen2ForCausalLM"]
        cfg = cls(
            architecture=str(arch[0]),
            model_type="qwen2",
            vocab_size=int(d["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(d["intermediate_size"]),
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            max_position_embeddings=int(d["max_position_embeddings"]),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_ids=_eos_tuple(d.get("eos_token_id")),
            initializer_range=float(d.get("initializer_range", 0.02)),
        )
        if min(cfg.vocab_size, cfg.intermediate_size, cfg.num_hidden_layers, cfg.max_position_embeddings) <= 0:
            raise ConfigError("invalid model sizes: vocabulary, intermediate size, layers and positions must be positive")
        if not (cfg.rms_norm_eps > 0 and cfg.rope_theta > 0):
            raise ConfigError("rms_norm_eps and rope_theta must be positive")
        return cfg

    @classmethod
    def read(cls, folder) -> "Qwen2Config":
        """Read ``config.json``; ``generation_config.json`` may override the EOS ids
        (flow_engine/config.py:54-62).  Sampling recipes are not imported."""
        folder = Path(folder)
        cfg = cls.from_dict(json.loads((folder / "config.json").read_text()))
        generation = folder / "generation_config.json"
        if generation.exists():
            eos = json.loads(generation.read_text()).get("eos_token_id")
            if eos is not None:
                cfg = replace(cfg, eos_token_ids=_eos_tuple(eos))
        return cfg

    # ---- derived ------------------------------------------------------
    def to_json_dict(self) -> dict:
        """The config.json that describes this configuration."""
        d = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "use_sliding_window": False,
            "initializer_range": self.initializer_range,
            "torch_dtype": "bfloat16",
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d
