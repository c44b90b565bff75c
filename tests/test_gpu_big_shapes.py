"""The layer sizes of the benchmark configuration (Qwen2.5-7B: hidden 3584, 28 query / 4 key-value heads
of size 128, intermediate 18944) with two layers and a shortened vocabulary, float32 and bfloat16, against
the plain implementation: a whole prompt, and most of it at once with the last tokens one by one.  Sizes
like these reach code that the tiny models do not: split matrix products, clustered norms, many key tiles."""
import numpy as np
import pytest

from helpers import plain_logits, random_tokens, replay_in_process, schedule_tail, schedule_whole
import tessweave_engine_b200 as tw

pytestmark = pytest.mark.gpu

BIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 20000, "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 2,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 32768,
    "tie_word_embeddings": False, "use_sliding_window": False, "hidden_act": "silu", "initializer_range": 0.02,
}


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    folder = tw.write_random_model(tmp_path_factory.mktemp("big") / "m", BIG, seed=5)
    tokens = random_tokens(BIG["vocab_size"], 150, 21)
    return folder, tokens, plain_logits(folder, tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_sizes_against_plain(dtype, big, tmp_path):
    folder, tokens, want = big
    tol = 1e-4 if dtype == "float32" else 0.03 * max(1.0, float(np.abs(want).max()))
    for name, steps in (("whole", schedule_whole({"r": tokens})), ("tail", schedule_tail({"r": tokens}, tail=10))):
        rows = replay_in_process(folder, dtype, steps, tmp_path / name)
        worst = max(float(np.abs(rows[("r", p)] - want[p]).max()) for p in range(len(tokens)))
        assert worst <= tol, f"{dtype} {name}: off by {worst:.3e} (logits up to {np.abs(want).max():.2f})"
