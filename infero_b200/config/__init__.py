from .spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                   ScheduleEntry)
from .qwen2 import ConfigError, Qwen2Config
from .engine_config import EngineConfig

__all__ = ["BlockSpec", "FeedForwardSpec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec",
           "ScheduleEntry", "ConfigError", "Qwen2Config", "EngineConfig"]
