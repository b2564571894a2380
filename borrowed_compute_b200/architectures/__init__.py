from . import fegidra, fudelorn, llama, logirax, pozirax  # noqa: F401  (registers Fegidra, Fudelorn, LlamaForCausalLM, Logirax, Pozirax)
from .registry import Architecture, architecture_names, register_architecture, resolve, unregister_architecture

__all__ = ["Architecture", "architecture_names", "register_architecture", "resolve", "unregister_architecture"]
