"""Weights: safetensors by tensor name, and the random-weights mode."""
from .loader import WeightError, fill_weights, load_model, parse_dtype
from .random_init import fill_random, write_random_model

__all__ = ["WeightError", "fill_weights", "load_model", "parse_dtype", "fill_random", "write_random_model"]
