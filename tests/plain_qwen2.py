"""A plain, slow implementation of the Qwen2 dense decoder, for tests only.

Whole sequences, no cache, no batching, one function for each part, fp32 on the
CPU by default.  It shares no code with the engine: it reads a model folder with
``safetensors`` directly and computes with elementary torch operations.  Every
function is written from the reference's formulas and cites them
(paths relative to the reference project).

``tests/golden/make_golden.py`` compared this file once with the reference's own
model code (``flow_engine.model.CausalLM``) on tiny random models and committed the
reference's logits; ``tests/test_plain.py`` checks against those files.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open


# ---------------------------------------------------------------------------
# reading a model folder
# ---------------------------------------------------------------------------
def read_folder(folder, dtype=torch.float32):
    """config.json as a dict and every tensor of model.safetensors, widened to ``dtype``."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as f:
        for key in f.keys():
            weights[key] = f.get_tensor(key).to(dtype)
    return config, weights


def sizes(config):
    """Sizes with the reference's defaults (flow_engine/config.py:38-48)."""
    hidden = int(config["hidden_size"])
    heads = int(config["num_attention_heads"])
    kv_heads = int(config.get("num_key_value_heads", heads))
    head_dim = int(config.get("head_dim", hidden // heads))
    return {
        "hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim,
        "layers": int(config["num_hidden_layers"]), "vocab": int(config["vocab_size"]),
        "eps": float(config.get("rms_norm_eps", 1e-6)), "theta": float(config.get("rope_theta", 10000.0)),
        "tied": bool(config.get("tie_word_embeddings", False)),
    }


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------
def embed(weights, tokens):
    """x = embed_tokens[ids], no scaling (flow_engine/model.py:100,176)."""
    return weights["model.embed_tokens.weight"][torch.as_tensor(tokens, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """x * rsqrt(mean(x^2, -1) + eps) * weight, statistics in fp32 (flow_engine/model.py:21-23)."""
    f = x.float()
    return (f * torch.rsqrt(f.square().mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


def linear(x, weight, bias=None):
    """y = x W^T + b with W stored [out, in] (nn.Linear; flow_engine/model.py:39-43)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def rope(x, positions, theta):
    """Rotate-half rotary encoding over the whole head (flow_engine/model.py:26-33).

    x: [T, heads, D]; inv[i] = theta ** (-(2i)/D); angle = position * inv; the pair of
    feature j is j + D/2: x' = x * cos + cat(-x[D/2:], x[:D/2]) * sin.
    """
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d, 2, dtype=torch.float32) / d)
    freq = torch.as_tensor(positions).float()[:, None] * inv
    freq = torch.cat((freq, freq), -1)[:, None, :]
    half = d // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), -1)
    return x * freq.cos().to(x.dtype) + rotated * freq.sin().to(x.dtype)


def attention_scores(q, k, window=None):
    """Scaled scores with the causal mask: key p is visible to the query at position t iff
    p <= t (flow_engine/model.py:196-198); scale D^-0.5 (SDPA default, model.py:199;
    kernels/paged_decode.py:34).  A window additionally hides keys p <= t - window.
    q: [heads, T, D], k: [heads, T, D] (already expanded to the query heads)."""
    t = q.shape[1]
    s = (q @ k.transpose(1, 2)) * (q.shape[-1] ** -0.5)
    pos = torch.arange(t)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    return s.masked_fill(~visible[None], float("-inf"))


def attention(q, k, v, window=None):
    """softmax(scores) @ v per query head; query head h uses key/value head h // (Hq / Hkv)
    (repeat_interleave, flow_engine/model.py:193-195).  q: [T, Hq, D], k/v: [T, Hkv, D]."""
    repeat = q.shape[1] // k.shape[1]
    kk = k.repeat_interleave(repeat, dim=1).transpose(0, 1)
    vv = v.repeat_interleave(repeat, dim=1).transpose(0, 1)
    probs = torch.softmax(attention_scores(q.transpose(0, 1), kk, window).float(), dim=-1).to(q.dtype)
    return (probs @ vv).transpose(0, 1)


def attention_layer(weights, prefix, x, positions, sz, window=None):
    """q/k/v projections with bias, rope on q and k, attention, unbiased output projection
    (flow_engine/model.py:39-43,183-186,201)."""
    t = x.shape[0]
    q = linear(x, weights[f"{prefix}.q_proj.weight"], weights[f"{prefix}.q_proj.bias"])
    k = linear(x, weights[f"{prefix}.k_proj.weight"], weights[f"{prefix}.k_proj.bias"])
    v = linear(x, weights[f"{prefix}.v_proj.weight"], weights[f"{prefix}.v_proj.bias"])
    q = rope(q.reshape(t, sz["heads"], sz["head_dim"]), positions, sz["theta"])
    k = rope(k.reshape(t, sz["kv_heads"], sz["head_dim"]), positions, sz["theta"])
    v = v.reshape(t, sz["kv_heads"], sz["head_dim"])
    out = attention(q, k, v, window).reshape(t, sz["heads"] * sz["head_dim"])
    return linear(out, weights[f"{prefix}.o_proj.weight"])


def swiglu(weights, prefix, x):
    """down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z), no biases (flow_engine/model.py:76-80)."""
    gate = linear(x, weights[f"{prefix}.gate_proj.weight"])
    up = linear(x, weights[f"{prefix}.up_proj.weight"])
    return linear(gate * torch.sigmoid(gate) * up, weights[f"{prefix}.down_proj.weight"])


def decoder_layer(weights, i, x, positions, sz):
    """x = x + attn(norm(x)); x = x + mlp(norm(x)) (flow_engine/model.py:179-202)."""
    p = f"model.layers.{i}"
    h = rms_norm(x, weights[f"{p}.input_layernorm.weight"], sz["eps"])
    x = x + attention_layer(weights, f"{p}.self_attn", h, positions, sz)
    h = rms_norm(x, weights[f"{p}.post_attention_layernorm.weight"], sz["eps"])
    return x + swiglu(weights, f"{p}.mlp", h)


def head(weights, x, sz):
    """logits = norm(x) @ W_lm^T in fp32; W_lm is the embedding when tied (flow_engine/model.py:110-112,204)."""
    y = rms_norm(x, weights["model.norm.weight"], sz["eps"])
    w = weights["model.embed_tokens.weight"] if sz["tied"] else weights["lm_head.weight"]
    return linear(y, w).float()


# ---------------------------------------------------------------------------
# whole model
# ---------------------------------------------------------------------------
@torch.no_grad()
def logits_of(config, weights, tokens):
    """fp32 logits [len(tokens), vocab] of one whole sequence."""
    sz = sizes(config)
    positions = list(range(len(tokens)))
    x = embed(weights, tokens)
    for i in range(sz["layers"]):
        x = decoder_layer(weights, i, x, positions, sz)
    return head(weights, x, sz)


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------
_MASK = (1 << 64) - 1


def uniform(seed: int, counter: int) -> float:
    """The engine's counter-based uniform: splitmix64 of seed + (counter + 1) * golden ratio,
    top 24 bits.  (The reference draws with torch.multinomial from a seeded CPU generator,
    flow_engine/engine.py:157-158; a device cannot reproduce that stream, so the engine
    defines this one and the test restates it here from the definition.)"""
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0


def choose(logits, temperature: float, seed: int = 0, counter: int = 0) -> int:
    """Greedy: the largest logit, lowest index at a tie (flow_engine/engine.py:155-156).
    Temperature: e = exp((x - max) / T); the first index whose running sum of e exceeds
    uniform(seed, counter) * sum(e)."""
    x = torch.as_tensor(logits, dtype=torch.float32)
    if temperature == 0:
        return int(torch.argmax(x))
    e = torch.exp((x - x.max()) / torch.tensor(temperature, dtype=torch.float32))
    c = torch.cumsum(e, 0)
    target = torch.tensor(uniform(seed, counter), dtype=torch.float32) * c[-1]
    idx = int(torch.searchsorted(c, target, right=True))
    return min(idx, x.numel() - 1)


@torch.no_grad()
def generate(config, weights, prompt, max_tokens, temperature=0.0, seed=0, eos=()):
    """Uncached generation: the whole sequence is recomputed for every token
    (as tests/test_engine.py:41-49 does with its library model)."""
    tokens, out = list(prompt), []
    for step in range(max_tokens):
        token = choose(logits_of(config, weights, tokens)[-1], temperature, seed, step)
        tokens.append(token)
        out.append(token)
        if token in eos:
            break
    return out
