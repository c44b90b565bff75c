"""Description of a model as data: which parts, with which parameters, in which order."""
from __future__ import annotations

from dataclasses import dataclass

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One block and the checkpoint prefix of its weights."""
    block: PartSpec
    prefix: str


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_of`` names an earlier schedule entry whose cache this run
    reads instead of writing one of its own; ``None`` gives the run its own cache."""
    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]      # the order in which layers run; a layer may appear twice
    embedding: PartSpec
    embedding_prefix: str                     # its weights are "<prefix>.<name the part declares>"
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
    tie_word_embeddings: bool                 # the head shares the embedding's matrix; the checkpoint has no tensor for it
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()
    init_std: float = 0.02
    ignored_suffixes: tuple[str, ...] = ()    # checkpoint tensors that are derived, not weights

    def __post_init__(self):
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, but there are {len(self.layers)} layers")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"schedule entry {i} may only read the cache of an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} must name the entry that owns the cache")
