"""The Qwen2 dense decoder as a ``ModelSpec``.

Layer kinds, constants and weight names follow flow_engine/model.py:36-112: GQA
attention with biased q/k/v and an unbiased output projection, rotate-half RoPE
over the whole head, RMSNorm before each sub-layer, SwiGLU, a final RMSNorm and an
output matrix that may be tied to the embedding.  ``rotary_emb.inv_freq`` tensors
in a checkpoint are derived values and are skipped (flow_engine/model.py:141-142).
"""
from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry

QWEN2_LAYER_NAMES = {"norm1": "input_layernorm", "mixer": "self_attn",
                     "norm2": "post_attention_layernorm", "feed_forward": "mlp"}


def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    mixer = PartSpec("gqa_attention", {
        "hidden": cfg.hidden_size, "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim, "qkv_bias": True, "out_bias": False, "window": None,
        "position": PartSpec("rope", {"theta": cfg.rope_theta})})
    ffn = PartSpec("swiglu", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size})
    block = PartSpec("pre_norm", {"hidden": cfg.hidden_size, "norm1": norm, "mixer": mixer, "norm2": norm,
                                  "feed_forward": ffn, "names": QWEN2_LAYER_NAMES})
    n = cfg.num_hidden_layers
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        layers=tuple(LayerSpec(block, f"model.layers.{i}") for i in range(n)),
        schedule=tuple(ScheduleEntry(i) for i in range(n)),
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size}),
        embedding_prefix="model.embed_tokens", final_norm=norm, final_norm_prefix="model.norm",
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size}), head_prefix="lm_head",
        tie_word_embeddings=cfg.tie_word_embeddings,
        max_position_embeddings=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids,
        init_std=cfg.initializer_range, ignored_suffixes=("rotary_emb.inv_freq",))


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_spec, model_type="qwen2")
