"""Weights from safetensors, by tensor name.

The model declares every tensor it wants (name, shape, role, destination); the
loader walks the checkpoint's shards, copies each named tensor into its
destination and reports *all* problems at once: missing tensors, unexpected ones,
duplicates and wrong shapes.  Matrices are kept in the run's element type,
vectors in fp32, integer tables in int32.  No pickle is read and no code of the
checkpoint runs.  Reference: flow_engine/model.py:114-159.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open

from ..config.registry import resolve_folder
from ..models.model import Model
from ..parts.base import Runtime


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every mismatch."""


def shard_names(folder: Path) -> list[str]:
    """``model.safetensors`` or the shards of ``model.safetensors.index.json``; names must be
    plain ``*.safetensors`` basenames (flow_engine/model.py:127-136)."""
    index = folder / "model.safetensors.index.json"
    if index.exists():
        names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    else:
        names = ["model.safetensors"]
    for name in names:
        if Path(name).name != name or not name.endswith(".safetensors"):
            raise WeightError(f"unsafe or unsupported shard filename {name!r}")
        if not (folder / name).exists():
            raise WeightError(f"{folder} holds no {name}")
    return names


def fill_weights(model: Model, folder) -> None:
    """Copy the checkpoint's tensors into the model's storage; one error names every fault."""
    folder = Path(folder).resolve(strict=True)
    decls = model.weight_decls()
    spec = model.spec
    redundant = model.redundant_names()
    seen: set[str] = set()
    unexpected, duplicate, wrong_shape = [], [], []
    for shard in shard_names(folder):
        with safe_open(str(folder / shard), framework="pt", device="cpu") as f:
            for key in f.keys():
                if key in redundant:
                    continue
                if any(key.endswith(sfx) for sfx in spec.ignored_suffixes):
                    continue
                decl = decls.get(key)
                if decl is None:
                    unexpected.append(key)
                    continue
                if key in seen:
                    duplicate.append(key)
                    continue
                seen.add(key)
                shape = tuple(f.get_slice(key).get_shape())
                if shape != tuple(decl.shape):
                    wrong_shape.append(f"{key}: checkpoint {list(shape)}, model {list(decl.shape)}")
                    continue
                tensor = f.get_tensor(key)
                if decl.role == "table_int" and tensor.dtype.is_floating_point:
                    wrong_shape.append(f"{key}: an integer table is expected, checkpoint holds {tensor.dtype}")
                    continue
                with torch.no_grad():
                    # casts to the destination's type and moves to its device; a destination may be a
                    # strided view of a packed buffer with the same elements in another shape
                    decl.dest.copy_(tensor.view(decl.dest.shape))
    missing = sorted(set(decls) - seen)
    if missing or unexpected or duplicate or wrong_shape:
        parts = [f"checkpoint {folder} does not fit architecture {spec.architecture}:"]
        if missing:
            parts.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if duplicate:
            parts.append(f"  duplicate ({len(duplicate)}): " + ", ".join(sorted(duplicate)))
        if wrong_shape:
            parts.append(f"  wrong shape ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        raise WeightError("\n".join(parts))
    model.finalize()


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("the engine runs in bfloat16 or float32")
        return dtype
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
    if dtype not in table:
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}")
    return table[dtype]


def load_model(folder, dtype="bfloat16", device="cuda") -> Model:
    """Model folder (config.json + safetensors) -> a model with its weights on ``device``.

    The class of the model is chosen by config.json through the architecture registry; the
    configuration is validated before any weight is read.
    """
    folder = Path(folder).resolve(strict=True)
    cfg, spec = resolve_folder(folder)
    runtime = Runtime(torch.device(device), parse_dtype(dtype))
    model = Model(spec, runtime, config=cfg)
    fill_weights(model, folder)
    return model
