from .base import (ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry)
from .qwen3 import ARCHITECTURE as QWEN3_ARCHITECTURE
from .qwen3 import Qwen3Config
from .registry import (config_class_for, known_architectures, load_config,
                       register_architecture)

register_architecture(QWEN3_ARCHITECTURE, Qwen3Config)

__all__ = ["ConfigError", "LayerSpec", "ModelPlan", "PartSpec", "ScheduleEntry", "Qwen3Config",
           "config_class_for", "known_architectures", "load_config", "register_architecture"]
