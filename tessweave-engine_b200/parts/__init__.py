"""Parts a model is put together from: embeddings, norms, position encodings, mixers,
feed-forwards, their arrangement in a block, and output heads."""
from .base import (Block, Embedding, FeedForward, FixedState, Head, Mixer, Norm, PagedKV, PagedView, Part, PartSpec,
                   PositionEncoding, ResidualStream, Runtime, SplitSum, StateView, StepContext, WeightDecl, Workspace,
                   build_part, dense_delta, register_part, registered)
from . import embedding, norms, positions, attention, feedforward, block, heads  # noqa: F401  (register the built-in kinds)

__all__ = ["Block", "Embedding", "FeedForward", "FixedState", "Head", "Mixer", "Norm", "PagedKV", "PagedView", "Part",
           "PartSpec", "PositionEncoding", "ResidualStream", "Runtime", "SplitSum", "StateView", "StepContext",
           "WeightDecl", "Workspace", "build_part", "dense_delta", "register_part", "registered"]
