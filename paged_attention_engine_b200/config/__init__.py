from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .engine_config import EngineConfig
from .errors import ConfigError
from .qwen2 import Qwen2Config
from .registry import ARCHITECTURES, Architecture, register_architecture, resolve, resolve_folder

__all__ = [
    "ARCHITECTURES", "Architecture", "ConfigError", "EngineConfig", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config",
    "ScheduleEntry", "register_architecture", "resolve", "resolve_folder",
]
