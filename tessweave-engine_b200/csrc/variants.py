"""Which compile-time variants of each CUDA source exist.

Most sources compile once.  Sources that are specialised by a macro (for instance the
head size of an attention kernel) are compiled for the sizes a model needs when the model
is built; ``default_variants`` lists what a full build compiles ahead of time.
"""
from __future__ import annotations

COMMON_HEAD_DIMS = (16, 32, 64, 128)

_SPECIALISED: dict[str, list[dict]] = {
    "attention_bf16": [{"TW_HEAD_DIM": d} for d in COMMON_HEAD_DIMS],
    "attention_tcgen05": [{"TW_HEAD_DIM": d} for d in (64, 128)],
    "attention_decode_tma": [{"TW_HEAD_DIM": d} for d in (64, 128)],
}


def specialise(name: str, variants: list[dict]) -> None:
    _SPECIALISED[name] = variants


def default_variants(name: str) -> list[dict]:
    return _SPECIALISED.get(name, [{}])
