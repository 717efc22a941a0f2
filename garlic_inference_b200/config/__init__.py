from .base import (ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry)
from .dugopel import ARCHITECTURE as DUGOPEL_ARCHITECTURE
from .dugopel import DugopelConfig
from .fivitar import ARCHITECTURE as FIVITAR_ARCHITECTURE
from .fivitar import FivitarConfig
from .kenovik import ARCHITECTURE as KENOVIK_ARCHITECTURE
from .kenovik import KenovikConfig
from .qwen3 import ARCHITECTURE as QWEN3_ARCHITECTURE
from .qwen3 import Qwen3Config
from .zogulorn import ARCHITECTURE as ZOGULORN_ARCHITECTURE
from .zogulorn import ZogulornConfig
from .registry import (architecture_name, config_class_for, known_architectures, load_config,
                       register_architecture)

register_architecture(QWEN3_ARCHITECTURE, Qwen3Config)
register_architecture(FIVITAR_ARCHITECTURE, FivitarConfig)
register_architecture(ZOGULORN_ARCHITECTURE, ZogulornConfig)
register_architecture(DUGOPEL_ARCHITECTURE, DugopelConfig)
register_architecture(KENOVIK_ARCHITECTURE, KenovikConfig)

__all__ = ["ConfigError", "LayerSpec", "ModelPlan", "PartSpec", "ScheduleEntry", "Qwen3Config", "FivitarConfig", "ZogulornConfig", "DugopelConfig", "KenovikConfig",
           "architecture_name", "config_class_for", "known_architectures", "load_config", "register_architecture"]
