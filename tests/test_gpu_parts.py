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
from tessweave_engine_b200.parts import (Embedding, FeedForward, FixedState, Head, Mixer, PartSpec, PositionEncoding,
                                         ResidualStream, Runtime, StateView, StepContext, WeightDecl, Workspace,
                                         build_part, dense_delta, register_part)
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

    seen_upcoming = []

    def forward(self, ctx, h, cache, write_cache):
        assert isinstance(cache, StateView)
        self.seen_upcoming.append(ctx.upcoming_weights)     # what the block says the part after this one streams first
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


@register_part("embedding", "toy_scaled_embedding")
class ToyScaledEmbedding(Embedding):
    """resid = weight[token] * scale + learned_position[position]: an embedding scale and absolute positions
    added to the stream, neither of which the built-in embedding has."""
    graph_safe = False

    def __init__(self, runtime, vocab, hidden, scale, max_positions):
        super().__init__(runtime)
        self.vocab, self.hidden, self.scale, self.max_positions = vocab, hidden, scale, max_positions
        self.weight = runtime.empty(vocab, hidden)
        self.positions = runtime.empty(max_positions, hidden)

    def weights(self):
        return [WeightDecl("weight", (self.vocab, self.hidden), dest=self.weight),
                WeightDecl("positions.weight", (self.max_positions, self.hidden), dest=self.positions)]

    def shared_matrix(self):
        return self.weight

    def forward(self, ctx):
        resid = ctx.workspace.get("toy.resid", (ctx.n_tokens, self.hidden), torch.float32)
        resid.copy_(self.weight[ctx.token_ids.long()].float() * self.scale + self.positions[ctx.positions.long()].float())
        return ResidualStream(resid)


@register_part("head", "toy_capped_head")
class ToyCappedHead(Head):
    """logits = cap * tanh((y @ W.T + bias) / cap): a bias and a cap, neither of which the built-in head has."""
    graph_safe = False

    def __init__(self, runtime, vocab, hidden, cap, tied=None):
        super().__init__(runtime)
        self.vocab, self.hidden, self.cap = vocab, hidden, cap
        self.tied = tied is not None
        self.weight = tied if tied is not None else runtime.empty(vocab, hidden)
        self.bias = runtime.empty(vocab, dtype=torch.float32)

    def weights(self):
        own = [] if self.tied else [WeightDecl("weight", (self.vocab, self.hidden), dest=self.weight)]
        return own + [WeightDecl("bias", (self.vocab,), role="vector", dest=self.bias)]

    def redundant_names(self):
        return ["weight"] if self.tied else []

    def forward(self, ctx, logits, y, n_rows):
        z = y[:n_rows].float() @ self.weight.float().t() + self.bias
        logits[:n_rows] = self.cap * torch.tanh(z / self.cap)


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
    # the toy feed-forward names no weight that it streams first, so the mixer before it was told of none;
    # the SwiGLU of the second layer names its gate/up matrix
    assert ToyDecayMixer.seen_upcoming and all(t is None for t in ToyDecayMixer.seen_upcoming)
    swiglu = model.blocks[1].feed_forward
    assert swiglu.streamed_first() is swiglu.w_gate_up and model.blocks[1].mixer.streamed_first() is None


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
    got = dense_delta(ctx, ffn.forward(ctx, x), dtype).float().cpu()
    w = {f"m.{d.name}": d.dest.float().cpu().reshape(d.shape) for d in ffn.weights()}
    assert torch.allclose(got, plain_qwen2.swiglu(w, "m", x.float().cpu()), **tol)


@pytest.mark.parametrize("tie", [True, False])
def test_toy_embedding_and_head_need_no_framework_change(tie):
    """A scaled embedding with learned positions and a biased, capped head -- registered here -- make a model
    whose first and last stage are not the built-in ones: ``Model`` only walks the parts its spec names.  Tied,
    the head shares the toy embedding's matrix and the checkpoint brings no tensor for it."""
    spec = spec_of([block(attention(position=PartSpec("none", {})))], [ScheduleEntry(0)],
                   embedding=PartSpec("toy_scaled_embedding", {"vocab": VOCAB, "hidden": H, "scale": 3.0, "max_positions": 128}),
                   head=PartSpec("toy_capped_head", {"vocab": VOCAB, "hidden": H, "cap": 2.5}), tie=tie)
    model, cache, runner, w = build(spec)
    assert ("head.weight" in w) == (not tie) and "head.bias" in w and "embed.positions.weight" in w
    assert not model.graph_safe
    if tie:
        assert model.head.weight.data_ptr() == model.embedding.weight.data_ptr() and model.redundant_names() == {"head.weight"}
    t = len(TOKENS)
    pos = list(range(t))
    x = w["embed.weight"][TOKENS] * 3.0 + w["embed.positions.weight"][:t]
    h = plain_qwen2.rms_norm(x, w["layers.0.n1.weight"], 1e-5)
    p = "layers.0.mix"
    q = plain_qwen2.linear(h, w[f"{p}.q_proj.weight"], w[f"{p}.q_proj.bias"]).reshape(t, HEADS, D)
    k = plain_qwen2.linear(h, w[f"{p}.k_proj.weight"], w[f"{p}.k_proj.bias"]).reshape(t, KV, D)
    v = plain_qwen2.linear(h, w[f"{p}.v_proj.weight"], w[f"{p}.v_proj.bias"]).reshape(t, KV, D)
    x = x + plain_qwen2.linear(plain_qwen2.attention(q, k, v).reshape(t, HEADS * D), w[f"{p}.o_proj.weight"])
    x = plain_swiglu(w, "layers.0", x)
    z = plain_qwen2.rms_norm(x, w["norm.weight"], 1e-5) @ w["embed.weight" if tie else "head.weight"].t() + w["head.bias"]
    want = 2.5 * torch.tanh(z / 2.5)
    for cuts in CUTS[:2]:
        assert float((run_cut(cache, runner, TOKENS, cuts) - want).abs().max()) <= 1e-4, cuts[:3]


def hand_made_context(rt, positions, seq_of_token, slots, q_start, q_len, kv_len):
    """A StepContext as the runner would stage it, for running one part outside a model."""
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    n = len(positions)
    return StepContext(runtime=rt, workspace=Workspace(torch.device("cuda")), n_tokens=n, n_seqs=len(slots),
                       token_ids=i32([0] * n), positions=i32(positions), seq_of_token=i32(seq_of_token),
                       seq_slot=i32(slots), seq_q_start=i32(q_start), seq_q_len=i32(q_len), seq_kv_len=i32(kv_len),
                       status=torch.zeros(1, dtype=torch.int32, device="cuda"), host_slot=slots, host_q_start=q_start,
                       host_q_len=q_len, host_kv_len=kv_len, max_q_len=max(q_len), max_kv_len=max(kv_len),
                       decode_only=all(c == 1 for c in q_len))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("head_dim,theta", [(16, 1e4), (64, 1e6), (24, 5e4)])
def test_position_encoding_alone(dtype, head_dim, theta):
    """``RotaryEmbedding.apply`` -- the interface every position encoding has -- against the plain rotation,
    for rows of several requests at scattered positions; the heads behind the first ``n_heads`` stay as they were."""
    rt = Runtime(torch.device("cuda"), dtype)
    rope = build_part("position", PartSpec("rope", {"theta": theta}), rt)
    positions = [0, 1, 2, 700, 3, 15, 16, 4095]
    ctx = hand_made_context(rt, positions, [0, 0, 0, 1, 2, 2, 2, 3], [0, 1, 2, 3], [0, 3, 4, 7], [3, 1, 3, 1], [3, 701, 17, 4096])
    heads, extra = 5, 2
    torch.manual_seed(4)
    x = torch.randn(len(positions), (heads + extra) * head_dim).to(dtype)
    qk = x.cuda().clone()
    rope.apply(ctx, qk, heads, head_dim)
    want = plain_qwen2.rope(x.float().reshape(len(positions), heads + extra, head_dim)[:, :heads], positions, theta)
    got = qk.float().cpu().reshape(len(positions), heads + extra, head_dim)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(got[:, :heads], want, **tol)
    assert torch.equal(got[:, heads:], x.float().reshape(len(positions), heads + extra, head_dim)[:, heads:])
    table = rope.fused_rotary_table(head_dim).cpu()
    assert torch.equal(table, theta ** (-torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


class TableHidden(PositionEncoding):
    """The rotary encoding behind the plain interface only: no table for a mixer to fuse."""

    def __init__(self, inner):
        super().__init__(inner.runtime)
        self.inner = inner

    def apply(self, ctx, qk, n_heads, head_dim):
        self.inner.apply(ctx, qk, n_heads, head_dim)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_alone(dtype):
    """The attention part built from its PartSpec and run on hand-made rows: a prompt portion of one request
    beside a single token of another whose keys are already in the cache (written by an earlier call of the
    same part).  With the position encoding's table hidden, the part must take ``apply`` and give the same."""
    rt = Runtime(torch.device("cuda"), dtype)
    hidden, heads, kv, d, page = 80, 4, 2, 32, 8
    spec = PartSpec("gqa_attention", {"hidden": hidden, "n_heads": heads, "n_kv_heads": kv, "head_dim": d, "qkv_bias": True,
                                      "position": PartSpec("rope", {"theta": 1e4})})
    results = []
    for hide_table in (False, True):
        mixer = build_part("mixer", spec, rt)
        torch.manual_seed(6)
        for decl in mixer.weights():
            decl.dest.copy_((torch.randn(decl.shape) * 0.15).view(decl.dest.shape))
        if hide_table:
            mixer.position = TableHidden(mixer.position)
        cache = tw.CacheManager([(mixer.cache_need(), None)], page, 12, 2, 64, dtype, rt.device, prefix_cache=False)
        a, b = cache.admit(None), cache.admit(None)
        torch.manual_seed(7)
        ha, hb = torch.randn(13, hidden) * 0.7, torch.randn(20, hidden) * 0.7
        # first call: b's first 19 rows (fills its cache); second call: 13 rows of a beside row 19 of b
        cache.ensure(b, 19); cache.sync_tables()
        ctx = hand_made_context(rt, list(range(19)), [0] * 19, [b.slot], [0], [19], [19])
        mixer.forward(ctx, hb[:19].to(dtype).cuda(), cache.view(0), True)
        cache.ensure(a, 13); cache.ensure(b, 20); cache.sync_tables()
        ctx = hand_made_context(rt, list(range(13)) + [19], [0] * 13 + [1], [a.slot, b.slot], [0, 13], [13, 1], [13, 20])
        h = torch.cat([ha, hb[19:]]).to(dtype).cuda()
        got = dense_delta(ctx, mixer.forward(ctx, h, cache.view(0), True), dtype).float().cpu()
        assert int(ctx.status) == 0
        results.append(got)
        w = {f"m.{decl.name}": decl.dest.float().cpu().reshape(decl.shape) for decl in mixer.weights()}
        sz = {"heads": heads, "kv_heads": kv, "head_dim": d, "theta": 1e4}
        for hs, rows in ((ha.to(dtype).float(), slice(0, 13)), (hb.to(dtype).float(), slice(13, 14))):
            t = hs.shape[0]
            q = plain_qwen2.rope(plain_qwen2.linear(hs, w["m.q_proj.weight"], w["m.q_proj.bias"]).reshape(t, heads, d), list(range(t)), 1e4)
            k = plain_qwen2.rope(plain_qwen2.linear(hs, w["m.k_proj.weight"], w["m.k_proj.bias"]).reshape(t, kv, d), list(range(t)), 1e4)
            v = plain_qwen2.linear(hs, w["m.v_proj.weight"], w["m.v_proj.bias"]).reshape(t, kv, d)
            want = plain_qwen2.linear(plain_qwen2.attention(q, k, v).reshape(t, heads * d), w["m.o_proj.weight"])
            want = want if rows.stop - rows.start == t else want[-1:]
            tol = dict(atol=5e-5, rtol=5e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
            assert torch.allclose(got[rows], want, **tol), (hide_table, rows)
    same = dict(atol=1e-6, rtol=0) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(results[0], results[1], **same)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts_alone(dtype):
    rt = Runtime(torch.device("cuda"), dtype)
    vocab, hidden = 211, 72
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab": vocab, "hidden": hidden}), rt)
    torch.manual_seed(8)
    emb.weight.copy_(torch.randn(vocab, hidden))
    ids = [0, 210, 5, 5, 99]
    ctx = hand_made_context(rt, [0, 1, 2, 3, 4], [0] * 5, [0], [0], [5], [5])
    ctx.token_ids = torch.tensor(ids, dtype=torch.int32, device="cuda")
    stream = emb.forward(ctx)
    assert stream.pending is None and stream.resid.dtype == torch.float32
    assert torch.equal(stream.resid, emb.weight[ids].float())
    for tied in (None, emb.shared_matrix()):
        head = build_part("head", PartSpec("linear_head", {"vocab": vocab, "hidden": hidden}), rt,
                          **({"tied": tied} if tied is not None else {}))
        assert (head.weights() == []) == (tied is not None) and head.redundant_names() == (["weight"] if tied is not None else [])
        if tied is None:
            head.weight.copy_(torch.randn(vocab, hidden) * 0.1)
        y = (torch.randn(7, hidden) * 0.5).to(dtype).cuda()
        logits = torch.full((9, vocab), float("nan"), device="cuda")
        head.forward(ctx, logits, y, 7)
        want = y.float() @ head.weight.float().t()
        assert logits.dtype == torch.float32 and torch.isnan(logits[7:]).all()
        assert torch.allclose(logits[:7], want, atol=2e-5 if dtype == torch.float32 else 2e-3, rtol=0)
    with pytest.raises(ValueError, match="tied head"):
        build_part("head", PartSpec("linear_head", {"vocab": vocab + 1, "hidden": hidden}), rt, tied=emb.shared_matrix())


def test_attention_shares_out_what_is_asked_into_l2(monkeypatch):
    """What a decode-only step asks into L2 ahead of its kernel: the attention kernel gets the head of the weights
    that the part after it streams first, its output product the part that follows; a short cache leaves all of it
    to the output product; a step that is not decode-only, or a block that announces nothing, asks for nothing."""
    for name in ("TESSWEAVE_WEIGHT_PREFETCH_MB", "TESSWEAVE_OUTPUT_PREFETCH_MB", "TESSWEAVE_WEIGHT_PREFETCH_MIN_KB"):
        monkeypatch.delenv(name, raising=False)
    rt = Runtime(torch.device("cuda"), torch.bfloat16)
    mixer = build_part("mixer", PartSpec("gqa_attention", {"hidden": 256, "n_heads": 4, "n_kv_heads": 2, "head_dim": 64,
                                                            "qkv_bias": True, "position": PartSpec("rope", {"theta": 1e4})}), rt)
    upcoming = torch.zeros(5000, 8192, dtype=torch.bfloat16, device="cuda")        # 78 MB
    mb = 1 << 20

    def plan(kv_len, q_len=1):
        ctx = hand_made_context(rt, [kv_len - 1] * q_len, [0] * q_len, [0], [0], [q_len], [kv_len])
        ctx.upcoming_weights = upcoming
        return ctx, mixer._prefetch_plan(ctx)

    ctx, (first, later) = plan(8192)                                   # 8,192 keys x 2 x 2 heads x 64 x 2 bytes = 4 MB
    assert first.data_ptr() == upcoming.data_ptr() and first.numel() * 2 == 24 * mb
    assert later.data_ptr() == upcoming.data_ptr() + 24 * mb and later.numel() * 2 == 24 * mb
    _, (first, later) = plan(512)                                      # 256 KB of cache: the kernel is too short
    assert first is None and later.data_ptr() == upcoming.data_ptr() and later.numel() * 2 == 24 * mb
    _, (first, later) = plan(8192, q_len=3)                            # a prompt portion: not the fused decode path
    assert first is None and later is None
    ctx.upcoming_weights = None
    assert mixer._prefetch_plan(ctx) == (None, None)
    monkeypatch.setenv("TESSWEAVE_OUTPUT_PREFETCH_MB", "70")           # more than is left: what there is
    _, (first, later) = plan(8192)
    assert later.numel() * 2 == upcoming.numel() * 2 - 24 * mb
    monkeypatch.setenv("TESSWEAVE_WEIGHT_PREFETCH_MB", "0")
    monkeypatch.setenv("TESSWEAVE_OUTPUT_PREFETCH_MB", "0")
    assert plan(8192)[1] == (None, None)
