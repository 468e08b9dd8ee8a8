from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from .registry import Architecture, architecture_names, register_architecture, resolve, unregister_architecture

__all__ = ["Architecture", "architecture_names", "register_architecture", "resolve", "unregister_architecture"]
