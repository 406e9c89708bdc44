from .base import ConfigError, ModelConfig, read_config_json, take
from .qwen3 import Qwen3Config
from .vemedra import VemedraConfig
from .pidutar import PidutarConfig
from .ledudra import LedudraConfig
from .tamovik import TamovikConfig
from .registry import (ArchitectureEntry, load_config, register_architecture,
                       registered_architectures, resolve_architecture)

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "VemedraConfig", "PidutarConfig", "LedudraConfig", "TamovikConfig", "read_config_json", "take",
           "ArchitectureEntry", "load_config", "register_architecture",
           "registered_architectures", "resolve_architecture"]
