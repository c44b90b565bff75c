"""Random weights: a model folder written from a configuration and a seed.

Every tensor is drawn on the CPU from its own generator, seeded by (seed, tensor
name), so any subset of tensors can be reproduced alone.  The rule per tensor is
the declaration's: matrices, embeddings and biases ~ N(0, std); norm weights
~ 1 + N(0, 0.1).  The reference has no such mode (its tests take random weights
from a library model: tests/test_engine.py:15-25).

``fill_random`` draws the same kind of weights straight into a model's device
storage, for sizes that one would not want to write to disk first.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from ..config.registry import resolve
from ..models.model import Model
from ..parts.base import Runtime, WeightDecl

NORM_WEIGHT_STD = 0.1


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def draw(decl: WeightDecl, seed: int, std: float) -> torch.Tensor:
    """The fp32 CPU tensor of one declaration."""
    g = torch.Generator(device="cpu").manual_seed(tensor_seed(seed, decl.name))
    if decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=torch.float32)
    if decl.role == "table_int":
        return torch.randint(0, 2 ** 15, decl.shape, generator=g, dtype=torch.int32)
    noise = torch.randn(decl.shape, generator=g, dtype=torch.float32)
    if decl.init == "one_plus_normal":
        return 1.0 + NORM_WEIGHT_STD * noise
    if decl.init == "normal":
        return std * noise
    raise ValueError(f"unknown init rule {decl.init!r} for {decl.name}")


def write_random_model(folder, config: dict, seed: int = 0, std: float | None = None,
                       store_dtype: str = "bfloat16") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (config.json contents).

    ``std`` defaults to the configuration's ``initializer_range``.  ``store_dtype`` is the
    element type in the file: with ``bfloat16`` every value is exactly representable in both
    run types, so a float32 run and a bfloat16 run start from the same numbers.
    """
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg, spec = resolve(config)
    if store_dtype not in ("bfloat16", "float32"):
        raise ValueError("store_dtype must be bfloat16 or float32")
    store = torch.bfloat16 if store_dtype == "bfloat16" else torch.float32
    std = spec.init_std if std is None else float(std)
    model = Model(spec, Runtime(torch.device("meta"), torch.float32), config=cfg)
    tensors = {}
    for name, decl in model.weight_decls().items():
        t = draw(decl, seed, std)
        tensors[name] = t if decl.role == "table_int" else t.to(store)
    out_cfg = dict(config)
    out_cfg.setdefault("architectures", [spec.architecture])
    out_cfg["torch_dtype"] = store_dtype
    (folder / "config.json").write_text(json.dumps(out_cfg, indent=2))
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt"})
    return folder


@torch.no_grad()
def fill_random(model: Model, seed: int = 0, std: float | None = None) -> Model:
    """Draw weights on the model's device (one generator stream per tensor)."""
    std = model.spec.init_std if std is None else float(std)
    device = model.runtime.device
    for name, decl in model.weight_decls().items():
        g = torch.Generator(device=device).manual_seed(tensor_seed(seed, name))
        if decl.init == "zeros":
            decl.dest.zero_()
            continue
        if decl.role == "table_int":
            decl.dest.copy_(torch.randint(0, 2 ** 15, decl.shape, generator=g, device=device, dtype=torch.int32))
            continue
        rows = decl.dest.shape[0]
        step = max(1, (64 << 20) // max(1, decl.dest[0].numel() if decl.dest.dim() > 1 else 1))
        for begin in range(0, rows, step):      # in slabs, so no second full-size copy is alive
            part = decl.dest[begin:begin + step]
            noise = torch.randn(part.shape, generator=g, device=device, dtype=torch.float32)
            part.copy_(1.0 + NORM_WEIGHT_STD * noise if decl.init == "one_plus_normal" else std * noise)
    model.finalize()
    return model
