"""A single-GPU inference engine for the Qwen2 dense decoder on NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token: typed configuration and
an architecture registry, weights from safetensors by name (or random), a model
assembled from parts, a paged cache manager, one step function over mixed batches,
a continuous-batching scheduler, sampling, and hand-written CUDA kernels.
"""
from .config import ConfigError, EngineConfig, Qwen2Config, register_architecture, resolve, resolve_folder
from .parts import PartSpec, register_part
from .models import LayerSpec, Model, ModelSpec, ScheduleEntry
from .weights import WeightError, fill_random, load_model, write_random_model
from .cache import CacheManager, CapacityError
from .engine.scheduler import Engine, Request
from .engine.runner import ModelRunner, StepEntry
from .engine.api import generate

__version__ = "0.1.0"

__all__ = ["ConfigError", "EngineConfig", "Qwen2Config", "register_architecture", "resolve", "resolve_folder",
           "PartSpec", "register_part", "LayerSpec", "Model", "ModelSpec", "ScheduleEntry", "WeightError",
           "fill_random", "load_model", "write_random_model", "CacheManager", "CapacityError", "Engine", "Request",
           "ModelRunner", "StepEntry", "generate"]
