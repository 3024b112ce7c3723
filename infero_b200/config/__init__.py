from .spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                   ScheduleEntry)
from .qwen2 import ConfigError, Qwen2Config
from .vufizen import VufizenConfig
from .gositar import GositarConfig
from .banelix import BanelixConfig
from .engine_config import EngineConfig

__all__ = ["BlockSpec", "FeedForwardSpec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec",
           "ScheduleEntry", "ConfigError", "Qwen2Config", "VufizenConfig", "GositarConfig", "BanelixConfig", "EngineConfig"]
