"""Parts alone, and the generality of their interfaces: a toy mixer with state of its own, a
toy feed-forward with routing and a toy position encoding are defined HERE, registered, built
into models and stepped, without a change to the framework's files.  A layer that runs twice, a
layer that reads another layer's cache and a windowed group with pages of its own are models
described as data and compared with plain computations."""
import math

import numpy as np
import pytest
import torch

import plain_qwen2
import tessweave_engine_b200 as tw
from tessweave_engine_b200.models import LayerSpec, Model, ModelSpec, ScheduleEntry
from tessweave_engine_b200.parts import (FeedForward, FixedState, Mixer, PartSpec, PositionEncoding, Runtime,
                                         StateView, WeightDecl, register_part)
from tessweave_engine_b200.engine.runner import ModelRunner, StepEntry

pytestmark = pytest.mark.gpu

H, HEADS, KV, D, INTER, VOCAB = 48, 3, 1, 16, 72, 97


# ---------------------------------------------------------------------------
# toy parts, defined in the test
# ---------------------------------------------------------------------------
@register_part("mixer", "toy_decay_state")
class ToyDecayMixer(Mixer):
    """state_t = decay * state_{t-1} + h_t;  delta_t = state_t @ W.T.  The state is a fixed-size
    per-request slot; it is carried across steps, so cutting must not change the result."""
    graph_safe = False

    def __init__(self, runtime, hidden, decay):
        super().__init__(runtime)
        self.hidden, self.decay = hidden, decay
        self.w = runtime.empty(hidden, hidden)

    def weights(self):
        return [WeightDecl("mix.weight", (self.hidden, self.hidden), dest=self.w)]

    def cache_need(self):
        return FixedState(self.hidden, torch.float32)

    def forward(self, ctx, h, cache, write_cache):
        assert isinstance(cache, StateView)
        out = ctx.workspace.get("toy.out", (ctx.n_tokens, self.hidden), self.runtime.dtype)
        for slot, start, count in zip(ctx.host_slot, ctx.host_q_start, ctx.host_q_len):
            state = cache.state[slot]
            rows = []
            for t in range(start, start + count):
                state = self.decay * state + h[t].float()
                rows.append(state)
            cache.state[slot] = state
            out[start:start + count] = (torch.stack(rows) @ self.w.float().t()).to(out.dtype)
        return out


@register_part("feed_forward", "toy_routed")
class ToyRoutedFeedForward(FeedForward):
    """Top-1 of ``experts`` small linear experts, router logits in fp32."""
    graph_safe = False

    def __init__(self, runtime, hidden, experts):
        super().__init__(runtime)
        self.hidden, self.experts = hidden, experts
        self.router = runtime.empty(experts, hidden)
        self.w = runtime.empty(experts, hidden, hidden)

    def weights(self):
        return [WeightDecl("router.weight", (self.experts, self.hidden), dest=self.router),
                WeightDecl("experts.weight", (self.experts, self.hidden, self.hidden), dest=self.w)]

    def forward(self, ctx, h):
        choice = (h.float() @ self.router.float().t()).argmax(-1)
        out = ctx.workspace.get("toy.ffn", (ctx.n_tokens, self.hidden), self.runtime.dtype)
        out.copy_(torch.einsum("nh,noh->no", h.float(), self.w.float()[choice]).to(out.dtype))
        return out


@register_part("position", "toy_scale")
class ToyScalePositions(PositionEncoding):
    """q and k are scaled by 1 / (1 + position / 64): not a rotation, so the generic path of the
    attention part (bias, then this, then the cache write) is what runs."""

    def apply(self, ctx, qk, n_heads, head_dim):
        scale = 1.0 / (1.0 + ctx.positions.float() / 64.0)
        cols = n_heads * head_dim
        qk[:, :cols] = (qk[:, :cols].float() * scale[:, None]).to(qk.dtype)


# ---------------------------------------------------------------------------
# model descriptions as data
# ---------------------------------------------------------------------------
NORM = PartSpec("rmsnorm", {"size": H, "eps": 1e-5})
NAMES = {"norm1": "n1", "mixer": "mix", "norm2": "n2", "feed_forward": "ff"}


def attention(window=None, position=None):
    return PartSpec("gqa_attention", {"hidden": H, "n_heads": HEADS, "n_kv_heads": KV, "head_dim": D, "qkv_bias": True,
                                      "window": window, "position": position or PartSpec("rope", {"theta": 1e4})})


SWIGLU = PartSpec("swiglu", {"hidden": H, "intermediate": INTER})


def block(mixer, ffn=SWIGLU):
    return PartSpec("pre_norm", {"hidden": H, "norm1": NORM, "mixer": mixer, "norm2": NORM, "feed_forward": ffn,
                                 "names": NAMES})


def spec_of(blocks, schedule, embedding=None, head=None, tie=False):
    return ModelSpec(architecture="ToyForTests", vocab_size=VOCAB, hidden_size=H,
                     layers=tuple(LayerSpec(b, f"layers.{i}") for i, b in enumerate(blocks)),
                     schedule=tuple(schedule), embedding=embedding or PartSpec("token_embedding", {"vocab": VOCAB, "hidden": H}),
                     embedding_prefix="embed", final_norm=NORM, final_norm_prefix="norm",
                     head=head or PartSpec("linear_head", {"vocab": VOCAB, "hidden": H}), head_prefix="head",
                     tie_word_embeddings=tie,
                     max_position_embeddings=512, init_std=0.08)


def build(spec, dtype=torch.float32, page=8, pages=40, requests=3, graphs=False):
    model = Model(spec, Runtime(torch.device("cuda"), dtype))
    tw.fill_random(model, seed=3)
    cache = tw.CacheManager(model.cache_needs(), page, pages, requests, 256, dtype, model.runtime.device, prefix_cache=False)
    runner = ModelRunner(model, cache, 256, requests, cuda_graphs=graphs)
    weights = {k: d.dest.detach().float().cpu().reshape(d.shape) for k, d in model.weight_decls().items()}
    return model, cache, runner, weights


def run_cut(cache, runner, tokens, cuts):
    """Feed ``tokens`` of one request in portions ``cuts``; logits of every position."""
    lease = cache.admit(None)
    rows, done = [], 0
    for n in cuts:
        part = tokens[done:done + n]
        if not part:
            break
        cache.ensure(lease, done + len(part))
        rows.append(runner.step([StepEntry(lease.slot, part, done, list(range(len(part))))]).cpu().clone())
        done += len(part)
        cache.advance(lease, None, done)
    runner.check_status()
    cache.release(lease)
    cache.check_invariants()
    return torch.cat(rows)


# ---------------------------------------------------------------------------
# plain computations of the toy models (whole sequence, no cache)
# ---------------------------------------------------------------------------
def plain_attention_block(w, prefix, x, positions, window=None, keys_from=None, scale_positions=False):
    sz = {"heads": HEADS, "kv_heads": KV, "head_dim": D, "theta": 1e4}
    t = x.shape[0]
    h = plain_qwen2.rms_norm(x, w[f"{prefix}.n1.weight"], 1e-5)
    p = f"{prefix}.mix"
    q = plain_qwen2.linear(h, w[f"{p}.q_proj.weight"], w[f"{p}.q_proj.bias"]).reshape(t, HEADS, D)
    k = plain_qwen2.linear(h, w[f"{p}.k_proj.weight"], w[f"{p}.k_proj.bias"]).reshape(t, KV, D)
    v = plain_qwen2.linear(h, w[f"{p}.v_proj.weight"], w[f"{p}.v_proj.bias"]).reshape(t, KV, D)
    if scale_positions:
        s = 1.0 / (1.0 + torch.tensor(positions).float() / 64.0)
        q, k = q * s[:, None, None], k * s[:, None, None]
    else:
        q, k = plain_qwen2.rope(q, positions, 1e4), plain_qwen2.rope(k, positions, 1e4)
    if keys_from is not None:
        k, v = keys_from
    out = plain_qwen2.attention(q, k, v, window).reshape(t, HEADS * D)
    x = x + plain_qwen2.linear(out, w[f"{p}.o_proj.weight"])
    return x, (k, v)


def plain_swiglu(w, prefix, x):
    h = plain_qwen2.rms_norm(x, w[f"{prefix}.n2.weight"], 1e-5)
    return x + plain_qwen2.swiglu(w, f"{prefix}.ff", h)


def plain_head(w, x):
    return plain_qwen2.linear(plain_qwen2.rms_norm(x, w["norm.weight"], 1e-5), w["head.weight"])


TOKENS = [int(t) for t in torch.randint(0, VOCAB, (61,), generator=torch.Generator().manual_seed(12))]
CUTS = [[61], [7, 2, 13, 3, 2, 16, 1, 17], [1] * 61]


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_twice_and_layer_reading_anothers_cache(dtype):
    """Schedule: layer 0, layer 1, layer 0 again (own cache), layer 1 reading the cache of its first run.
    In bfloat16 the single-token steps go through the decode attention that makes q, k and v itself: the run
    that reads another run's cache must then rotate its query but write nothing."""
    spec = spec_of([block(attention()), block(attention())],
                   [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1)])
    model, cache, runner, w = build(spec, dtype=dtype)
    assert len(cache.groups) == 1 and cache.groups[0].k.shape[0] == 3         # three caches for four runs
    pos = list(range(len(TOKENS)))
    x = w["embed.weight"][TOKENS]
    x, _ = plain_attention_block(w, "layers.0", x, pos); x = plain_swiglu(w, "layers.0", x)
    x, kv1 = plain_attention_block(w, "layers.1", x, pos); x = plain_swiglu(w, "layers.1", x)
    x, _ = plain_attention_block(w, "layers.0", x, pos); x = plain_swiglu(w, "layers.0", x)
    x, _ = plain_attention_block(w, "layers.1", x, pos, keys_from=kv1); x = plain_swiglu(w, "layers.1", x)
    want = plain_head(w, x)
    tol = 1e-4 if dtype == torch.float32 else 0.03 * max(1.0, float(want.abs().max()))
    for cuts in CUTS:
        got = run_cut(cache, runner, TOKENS, cuts)
        assert float((got - want).abs().max()) <= tol, cuts[:3]


def test_window_group_has_pages_of_its_own_and_returns_them():
    """Layer 0 sees a window of 12 keys, layer 1 all keys: two groups, two block tables.  The
    windowed group gives pages back while the request runs; logits equal the plain windowed model."""
    spec = spec_of([block(attention(window=12)), block(attention())], [ScheduleEntry(0), ScheduleEntry(1)])
    model, cache, runner, w = build(spec, pages=12)
    assert len(cache.groups) == 2
    pos = list(range(len(TOKENS)))
    x = w["embed.weight"][TOKENS]
    x, _ = plain_attention_block(w, "layers.0", x, pos, window=12); x = plain_swiglu(w, "layers.0", x)
    x, _ = plain_attention_block(w, "layers.1", x, pos); x = plain_swiglu(w, "layers.1", x)
    want = plain_head(w, x)
    windowed = next(g for g in cache.groups if g.window == 12)
    for cuts in CUTS:
        cache.poison_freed = True
        got = run_cut(cache, runner, TOKENS, cuts)
        assert torch.isfinite(got).all()
        assert float((got - want).abs().max()) <= 1e-4, cuts[:3]
    # a second request while the first is long: the windowed group never holds more than its window's pages
    lease = cache.admit(None)
    done = 0
    for n in [5] * 12:
        cache.ensure(lease, done + n)
        runner.step([StepEntry(lease.slot, TOKENS[done:done + n], done, [])])
        done += n
        cache.advance(lease, None, done)
        gi = cache.groups.index(windowed)
        assert sum(p >= 0 for p in lease.tables[gi]) <= math.ceil((12 + 5) / 8) + 1
    cache.release(lease)
    assert len(windowed.free) == 12


def test_toy_position_encoding_takes_the_generic_path():
    spec = spec_of([block(attention(position=PartSpec("toy_scale", {})))], [ScheduleEntry(0)])
    model, cache, runner, w = build(spec)
    pos = list(range(len(TOKENS)))
    x = w["embed.weight"][TOKENS]
    x, _ = plain_attention_block(w, "layers.0", x, pos, scale_positions=True); x = plain_swiglu(w, "layers.0", x)
    want = plain_head(w, x)
    for cuts in CUTS[:2]:
        assert float((run_cut(cache, runner, TOKENS, cuts) - want).abs().max()) <= 1e-4


def test_toy_mixer_with_state_and_routed_feed_forward():
    """A model whose first layer is the toy state mixer with the toy routed feed-forward and whose
    second layer is attention + SwiGLU: state slots beside pages, one step function for both."""
    spec = spec_of([block(PartSpec("toy_decay_state", {"hidden": H, "decay": 0.9}),
                          PartSpec("toy_routed", {"hidden": H, "experts": 4})),
                    block(attention())], [ScheduleEntry(0), ScheduleEntry(1)])
    model, cache, runner, w = build(spec)
    assert not model.graph_safe and list(cache.state) == [0] and len(cache.groups) == 1
    x = w["embed.weight"][TOKENS]
    h = plain_qwen2.rms_norm(x, w["layers.0.n1.weight"], 1e-5)
    state, rows = torch.zeros(H), []
    for t in range(len(TOKENS)):
        state = 0.9 * state + h[t]
        rows.append(state)
    x = x + torch.stack(rows) @ w["layers.0.mix.mix.weight"].t()
    h = plain_qwen2.rms_norm(x, w["layers.0.n2.weight"], 1e-5)
    choice = (h @ w["layers.0.ff.router.weight"].t()).argmax(-1)
    x = x + torch.einsum("nh,noh->no", h, w["layers.0.ff.experts.weight"][choice])
    x, _ = plain_attention_block(w, "layers.1", x, list(range(len(TOKENS)))); x = plain_swiglu(w, "layers.1", x)
    want = plain_head(w, x)
    for cuts in CUTS:
        got = run_cut(cache, runner, TOKENS, cuts)
        assert float((got - want).abs().max()) <= 2e-4, cuts[:3]
    # two requests side by side keep their own state
    a, b = cache.admit(None), cache.admit(None)
    cache.ensure(a, 30); cache.ensure(b, 30)
    l1 = runner.step([StepEntry(a.slot, TOKENS[:10], 0, [9]), StepEntry(b.slot, TOKENS[20:23], 0, [2])]).cpu().clone()
    l2 = runner.step([StepEntry(b.slot, TOKENS[23:30], 3, [6]), StepEntry(a.slot, TOKENS[10:11], 10, [0])]).cpu().clone()
    assert float((l1[0] - want[9]).abs().max()) <= 2e-4 and float((l2[1] - want[10]).abs().max()) <= 2e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_builtin_parts_alone(dtype):
    """RMSNorm, SwiGLU and the attention part, each built from its PartSpec and run on its own."""
    from tessweave_engine_b200.parts import StepContext, Workspace, build_part
    rt = Runtime(torch.device("cuda"), dtype)
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    torch.manual_seed(9)
    n = 11
    # norm
    norm = build_part("norm", PartSpec("rmsnorm", {"size": 200, "eps": 1e-6}), rt)
    norm.weight.copy_(1 + 0.1 * torch.randn(200))
    resid = torch.randn(n, 200, device="cuda")
    out = torch.empty(n, 200, device="cuda", dtype=dtype)
    norm.forward(None, out, resid, None, n)
    assert torch.allclose(out.float().cpu(), plain_qwen2.rms_norm(resid.cpu(), norm.weight.cpu(), 1e-6), **tol)
    # feed-forward
    ffn = build_part("feed_forward", PartSpec("swiglu", {"hidden": 200, "intermediate": 136}), rt)
    for d in ffn.weights():
        d.dest.copy_((torch.randn(d.shape) * 0.1).view(d.dest.shape))
    x = (torch.randn(n, 200, device="cuda") * 0.5).to(dtype)
    ws = Workspace(torch.device("cuda"))
    ctx = type("Ctx", (), {"n_tokens": n, "workspace": ws,
                           "status": torch.zeros(1, dtype=torch.int32, device="cuda")})()
    got = ffn.forward(ctx, x).float().cpu()
    w = {f"m.{d.name}": d.dest.float().cpu().reshape(d.shape) for d in ffn.weights()}
    assert torch.allclose(got, plain_qwen2.swiglu(w, "m", x.float().cpu()), **tol)
