from .errors import CacheError, ConfigError, WeightsError
from .fegidra import FegidraConfig
from .llama import Llama3RopeScaling, LlamaConfig
from .pozirax import PoziraxConfig

__all__ = ["CacheError", "ConfigError", "WeightsError", "FegidraConfig", "Llama3RopeScaling", "LlamaConfig", "PoziraxConfig"]
