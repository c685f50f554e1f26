from .spec import (ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry)
from .qwen3 import Qwen3Config
from .nuvilorn import NuvilornConfig
from .zekazen import ZekazenConfig
from .lodevik import LodevikConfig
from .sudupel import SudupelConfig

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "Qwen3Config", "NuvilornConfig",
           "ZekazenConfig", "LodevikConfig", "SudupelConfig"]
