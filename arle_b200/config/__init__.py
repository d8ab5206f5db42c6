from .model_spec import ModelSpec, ScheduleEntry
from .kolodra import KolodraConfig
from .lasupel import LasupelConfig
from .lukinex import LukinexConfig
from .qwen3 import ConfigError, Qwen3Config
from .zuderax import ZuderaxConfig
from .registry import (UnknownArchitecture, config_class_for, config_from_dict, load_config,
                       register_architecture, registered_architectures)

register_architecture(Qwen3Config.architecture, Qwen3Config)
register_architecture(KolodraConfig.architecture, KolodraConfig)
register_architecture(ZuderaxConfig.architecture, ZuderaxConfig)
register_architecture(LasupelConfig.architecture, LasupelConfig)
register_architecture(LukinexConfig.architecture, LukinexConfig)

__all__ = ["ModelSpec", "ScheduleEntry", "ConfigError", "Qwen3Config", "KolodraConfig", "ZuderaxConfig", "LasupelConfig", "LukinexConfig", "UnknownArchitecture", "config_class_for",
           "config_from_dict", "load_config", "register_architecture", "registered_architectures"]
