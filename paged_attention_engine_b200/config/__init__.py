from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .qwen2 import ConfigError, Qwen2Config
from .registry import ARCHITECTURES, Architecture, register_architecture, resolve, resolve_folder

__all__ = [
    "ARCHITECTURES", "Architecture", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config",
    "ScheduleEntry", "register_architecture", "resolve", "resolve_folder",
]
