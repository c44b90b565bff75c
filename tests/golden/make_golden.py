"""Makes the golden files of this folder from the reference's own model code.

Run once, on the CPU, with the reference project importable:

    python tests/golden/make_golden.py /path/to/reference

For each tiny configuration it writes a random model folder (fp32 storage) into a
temporary folder with the engine's random-weights mode, loads it with the
reference's ``flow_engine.model.CausalLM.load`` (which also checks names and
shapes), runs the reference's forward over a fixed token sequence -- whole, and in
portions through its paged pool -- and stores the whole-sequence fp32 logits as
``qwen2_tiny_<name>.npy`` beside the token ids in ``qwen2_tiny_<name>.json``.  It then
prints how far the plain implementation of ``tests/plain_qwen2.py`` is from them.
``tests/test_plain.py`` rebuilds the same folders from the same seeds and compares.
"""
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

import plain_qwen2  # noqa: E402
from tiny_configs import CONFIGS, SEEDS  # noqa: E402
from tessweave_engine_b200 import write_random_model  # noqa: E402

LENGTHS = {"A": 33, "B": 40, "C": 29}


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from flow_engine.cache import KVPool
    from flow_engine.model import CausalLM

    torch.set_num_threads(2)
    for name, config in CONFIGS.items():
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(tmp, config, seed=SEEDS[name], store_dtype="float32")
            ref = CausalLM.load(tmp, "cpu", torch.float32)
            g = torch.Generator().manual_seed(SEEDS[name] + 1)
            tokens = torch.randint(0, config["vocab_size"], (LENGTHS[name],), generator=g).tolist()
            n = len(tokens)
            pool = KVPool(ref.config, 8, 16, torch.float32, "cpu")
            table = pool.allocate(4)
            with torch.inference_mode():
                whole = ref(torch.tensor([tokens]), torch.arange(n)[None], [table], [n], pool, all_logits=True)[0]
                pool2 = KVPool(ref.config, 8, 16, torch.float32, "cpu")
                table2 = pool2.allocate(4)
                cut = n // 2 + 3
                ref(torch.tensor([tokens[:cut]]), torch.arange(cut)[None], [table2], [cut], pool2)
                tail = ref(torch.tensor([tokens[cut:]]), torch.arange(cut, n)[None], [table2], [n], pool2,
                           all_logits=True)[0]
            print(name, "reference whole vs portions:", float((whole[cut:] - tail).abs().max()))
            cfg, weights = plain_qwen2.read_folder(tmp)
            mine = plain_qwen2.logits_of(cfg, weights, tokens)
            print(name, "plain vs reference, max abs:", float((mine - whole).abs().max()),
                  "| logits abs max:", float(whole.abs().max()))
            np.save(HERE / f"qwen2_tiny_{name}.npy", whole.numpy().astype(np.float32))
            (HERE / f"qwen2_tiny_{name}.json").write_text(json.dumps(
                {"config": config, "seed": SEEDS[name], "store_dtype": "float32", "tokens": tokens,
                 "made_by": "tests/golden/make_golden.py with flow_engine.model.CausalLM (reference 0.1.0a1), CPU fp32"}))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference project's checkout>")
    main(sys.argv[1])
