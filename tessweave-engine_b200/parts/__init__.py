"""Parts a model is put together from: norms, position encodings, mixers,
feed-forwards and their arrangement in a block."""
from .base import (Block, FeedForward, FixedState, Mixer, Norm, PagedKV, PagedView, Part, PartSpec,
                   PositionEncoding, ResidualStream, Runtime, StateView, StepContext, WeightDecl, Workspace,
                   build_part, register_part, registered)
from . import norms, positions, attention, feedforward, block  # noqa: F401  (register the built-in kinds)

__all__ = ["Block", "FeedForward", "FixedState", "Mixer", "Norm", "PagedKV", "PagedView", "Part", "PartSpec",
           "PositionEncoding", "ResidualStream", "Runtime", "StateView", "StepContext", "WeightDecl", "Workspace",
           "build_part", "register_part", "registered"]
