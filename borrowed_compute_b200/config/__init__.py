from .errors import CacheError, ConfigError, WeightsError
from .fegidra import FegidraConfig
from .fudelorn import FudelornConfig
from .logirax import LogiraxConfig
from .llama import Llama3RopeScaling, LlamaConfig
from .pozirax import PoziraxConfig

__all__ = ["CacheError", "ConfigError", "WeightsError", "FegidraConfig", "FudelornConfig", "Llama3RopeScaling", "LlamaConfig", "LogiraxConfig", "PoziraxConfig"]
