"""A small B200-native library for the Llama dense decoder: from a model folder to tokens.

    from borrowed_compute_b200 import Local, Sampling
    model = Local.load("path/to/folder")              # config.json + model.safetensors
    tokens, stats = model.generate([1, 2, 3], 64, Sampling(temperature=0.8, top_p=0.95, seed=7))
"""

from . import architectures, parts  # noqa: F401  (register the built-in architecture and parts)
from .architectures import register_architecture
from .config import CacheError, ConfigError, LlamaConfig, WeightsError
from .engine import Engine, Stats, StepEntry
from .local import Local
from .sampling import Sampling
from .weights import write_model_folder

__all__ = ["CacheError", "ConfigError", "Engine", "LlamaConfig", "Local", "Sampling", "Stats", "StepEntry", "WeightsError",
           "register_architecture", "write_model_folder"]
