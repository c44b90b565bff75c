"""Token selection: greedy and temperature sampling, defined once for device and host."""
from .sampler import choose_tokens, select_tokens, uniform

__all__ = ["choose_tokens", "select_tokens", "uniform"]
