"""A paged-attention inference engine for one B200: configuration, weights, parts, cache
manager, step function, scheduler, sampling and trace replay over hand-written CUDA."""

from .cache import AllocResult, AllocStatus, BlockAllocator, CacheManager, PagedKVCache
from .config import ConfigError, EngineConfig, Qwen2Config, register_architecture
from .engine.api import LLM
from .engine.batch import StepEntry
from .engine.executor import ModelExecutor
from .engine.llm import Engine
from .engine.scheduler import Event, EventKind, Request, Scheduler, Sequence, SequenceStatus, StepResult
from .weights import WeightsError, write_random_model

__all__ = [
    "AllocResult", "AllocStatus", "BlockAllocator", "CacheManager", "ConfigError", "Engine", "EngineConfig", "Event", "EventKind",
    "LLM", "ModelExecutor", "PagedKVCache", "Qwen2Config", "Request", "Scheduler", "Sequence", "SequenceStatus",
    "StepEntry", "StepResult", "WeightsError", "register_architecture", "write_random_model",
]
