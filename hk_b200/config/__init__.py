from .base import (ConfigError, ModelConfig, architecture_name, config_from_dict, load_config,
                   register_architecture, resolve_architecture, supported_architectures)
from .kedanex import KedanexConfig
from .mifolorn import MifolornConfig
from .padodra import PadodraConfig
from .qwen3 import Qwen3Config
from .zazulix import ZazulixConfig

__all__ = [
    "ConfigError", "KedanexConfig", "MifolornConfig", "ModelConfig", "PadodraConfig", "Qwen3Config", "ZazulixConfig", "architecture_name", "config_from_dict", "load_config",
    "register_architecture", "resolve_architecture", "supported_architectures",
]
