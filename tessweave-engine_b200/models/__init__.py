"""Models: a generic assembly of parts, and the architectures described with it."""
from .spec import LayerSpec, ModelSpec, ScheduleEntry
from .model import Model
from . import qwen2  # noqa: F401  (registers "Qwen2ForCausalLM")

__all__ = ["LayerSpec", "ModelSpec", "ScheduleEntry", "Model"]
