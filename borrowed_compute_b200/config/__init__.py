from .errors import CacheError, ConfigError, WeightsError
from .llama import Llama3RopeScaling, LlamaConfig

__all__ = ["CacheError", "ConfigError", "WeightsError", "Llama3RopeScaling", "LlamaConfig"]
