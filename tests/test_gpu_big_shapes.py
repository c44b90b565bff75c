"""The layer sizes of the benchmark configuration (Qwen2.5-7B: hidden 3584, 28 query / 4 key-value heads
of size 128, intermediate 18944) with two layers and a shortened vocabulary, float32 and bfloat16, against
the plain implementation: a whole prompt, and most of it at once with the last tokens one by one.  Sizes
like these reach code that the tiny models do not: split matrix products, clustered norms, many key tiles."""
import numpy as np
import pytest

from helpers import (note_error, plain_logits, random_tokens, replay_in_process, schedule_portions, schedule_tail,
                     schedule_whole)
import tessweave_engine_b200 as tw

pytestmark = pytest.mark.gpu

# bfloat16 bound relative to the largest logit: twice the worst difference observed on a B200 at these sizes
# (TESSWEAVE_ERROR_LOG=<file> records what every comparison saw)
BF16_RELATIVE = 0.03

BIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 20000, "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 2,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 32768,
    "tie_word_embeddings": False, "use_sliding_window": False, "hidden_act": "silu", "initializer_range": 0.02,
}


# The layer sizes of the two larger benchmark configurations (Qwen2.5-14B and 32B: hidden 5120, 40 query and
# 8 key/value heads, i.e. groups of five; intermediate 13,824 and 27,648), two layers each.  They take other routes
# than the 7B sizes: the 128-row tiles of the gate/up matrix do not balance over the SMs, so decode portions of 9 to
# 64 rows take the library's product and a separate SiLU.mul; the block-pair product is refused where its tiles
# do not fill whole rounds; the small-batch product gives a row tile to two warps.
def larger(intermediate):
    return {**BIG, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8,
            "intermediate_size": intermediate}


SIZES = {"7b": (BIG, 150), "14b": (larger(13824), 800), "32b": (larger(27648), 800)}


@pytest.fixture(scope="module", params=list(SIZES))
def big(request, tmp_path_factory):
    config, length = SIZES[request.param]
    folder = tw.write_random_model(tmp_path_factory.mktemp("big") / request.param, config, seed=5)
    tokens = random_tokens(config["vocab_size"], length, 21)
    return request.param, folder, tokens, plain_logits(folder, tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_sizes_against_plain(dtype, big, tmp_path):
    """Whole (for the larger sizes one portion of 800 rows: the prompt-sized products), most of it at once and the
    last ten tokens one by one (the small-batch products), and portions of 9 to 64 rows (the streaming products and
    the library's)."""
    size, folder, tokens, want = big
    scale = max(1.0, float(np.abs(want).max()))
    tol = 1e-4 if dtype == "float32" else BF16_RELATIVE * scale
    for name, steps in (("whole", schedule_whole({"r": tokens})), ("tail", schedule_tail({"r": tokens}, tail=10)),
                        ("portions", schedule_portions({"r": tokens}, sizes=(12, 40, 64, 9, 25)))):
        rows = replay_in_process(folder, dtype, steps, tmp_path / name)
        errs = np.array([float(np.abs(rows[("r", p)] - want[p]).max()) for p in range(len(tokens))])
        worst = float(errs.max())
        note_error("big_shapes", f"{size}/{dtype}/{name}", worst, scale)
        assert worst <= tol, (f"{size} {dtype} {name}: off by {worst:.3e} at position {int(errs.argmax())} "
                              f"({int((errs > tol).sum())} of {len(errs)} positions beyond {tol:.1e}, median {np.median(errs):.3e}; "
                              f"logits up to {np.abs(want).max():.2f})")


# A model whose prompt portions are long enough for the tcgen05 attention kernel (128 tokens and
# more, head size 64), small enough to replay several requests in many ways.
MEDIUM = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 1536, "hidden_size": 320, "intermediate_size": 704, "num_hidden_layers": 2,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 64,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 2048,
    "tie_word_embeddings": True, "use_sliding_window": False, "hidden_act": "silu", "initializer_range": 0.05,
}


@pytest.fixture(scope="module")
def medium(tmp_path_factory):
    folder = tw.write_random_model(tmp_path_factory.mktemp("medium") / "m", MEDIUM, seed=9)
    requests = {rid: random_tokens(MEDIUM["vocab_size"], n, 40 + i) for i, (rid, n) in enumerate(
        (("a", 420), ("b", 131), ("c", 300), ("d", 257), ("e", 64), ("f", 700)))}
    return folder, requests, {rid: plain_logits(folder, toks) for rid, toks in requests.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "tail", "portions", "mixed"])
def test_long_portions_against_plain(dtype, how, medium, tmp_path, monkeypatch):
    """Portions of 128 tokens and more beside short ones and single tokens: in bfloat16 the long ones run on
    the tcgen05 attention kernel and the others on the mma.sync kernels, and every position must still
    agree with the plain implementation, whichever kernel wrote its keys and read them.  Steps of more than
    64 rows take the gate/up product on block pairs here (forced: the product path takes the pairs only
    where their tiles fill the GPU, which this small model's do not)."""
    from helpers import schedule_mixed, schedule_portions
    monkeypatch.setenv("TESSWEAVE_PAIR_GEMM", "force")
    folder, requests, want = medium
    steps = {
        "whole": lambda: schedule_whole(requests),
        "tail": lambda: schedule_tail(requests, tail=8),
        "portions": lambda: schedule_portions(requests, sizes=(130, 2, 200, 1, 64, 129, 3, 256, 520)),
        "mixed": lambda: schedule_mixed(requests, live=4, seed=4, prefill=(140, 2, 128, 9, 190, 300), decode_from=0.9),
    }[how]()
    rows = replay_in_process(folder, dtype, steps, tmp_path / how)
    for rid, toks in requests.items():
        scale = max(1.0, float(np.abs(want[rid]).max()))
        tol = 1e-4 if dtype == "float32" else BF16_RELATIVE * scale
        got = [p for p in range(len(toks)) if (rid, p) in rows]
        assert got, f"no logits for request {rid}"
        worst = max(float(np.abs(rows[(rid, p)] - want[rid][p]).max()) for p in got)
        note_error("long_portions", f"{dtype}/{how}/{rid}", worst, scale)
        assert worst <= tol, f"{dtype} {how} request {rid}: off by {worst:.3e}"


@pytest.fixture(scope="module")
def model_7b(tmp_path_factory):
    folder = tw.write_random_model(tmp_path_factory.mktemp("graphs") / "7b", BIG, seed=6)
    return tw.load_model(folder, "bfloat16", "cuda")


@pytest.mark.parametrize("n_requests", [1, 3, 8])
def test_graph_steps_at_benchmark_sizes_equal_eager_steps(n_requests, model_7b):
    """Decode steps replayed from CUDA graphs launch every kernel with programmatic serialization: kernels are
    resident before the one before them has ended, the q/k/v product lets a small attention launch start early,
    and the attention, its output product and the gate/up product ask for later weights.  None of that may change
    a token: the same requests, generated with graphs and kernel by kernel, at the 7B layer sizes (the TMA decode
    attention, clusters, split products) and with a context long enough for every prefetch to be issued."""
    model = model_7b
    prompts = [random_tokens(BIG["vocab_size"], 30 + 7 * i, 90 + i) for i in range(n_requests)]
    outs = []
    for graphs in (True, False):
        cfg = tw.EngineConfig(block_size=16, kv_blocks=64 * n_requests + 8, max_context=1024, max_active=n_requests,
                              prefill_chunk=256, cuda_graphs=graphs)
        outs.append(tw.generate(model, prompts, max_tokens=16, ignore_eos=True, engine_config=cfg))
    assert outs[0] == outs[1]
    assert all(len(o) == 16 for o in outs[0])
