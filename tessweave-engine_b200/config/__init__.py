"""Typed configuration of model and engine, and the architecture registry."""
from .model_config import ConfigError, Qwen2Config
from .engine_config import EngineConfig
from .registry import architecture_of, architectures, register_architecture, resolve, resolve_folder

__all__ = ["ConfigError", "Qwen2Config", "EngineConfig", "architecture_of", "architectures",
           "register_architecture", "resolve", "resolve_folder"]
