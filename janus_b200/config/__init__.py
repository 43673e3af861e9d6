from .base import ConfigError, KeyReader, read_config_json
from .buludra import BuludraConfig
from .llama import LlamaConfig, RopeScaling
from .mugedra import MugedraConfig
from .ramolix import RamolixConfig
from .zivitar import ZivitarConfig
from .registry import (Architecture, architecture_name, register_architecture,
                       registered_architectures, resolve_architecture)

__all__ = [
    "ConfigError", "KeyReader", "read_config_json", "BuludraConfig", "LlamaConfig", "RopeScaling", "MugedraConfig", "RamolixConfig", "ZivitarConfig", "Architecture",
    "architecture_name", "register_architecture", "registered_architectures", "resolve_architecture",
]
