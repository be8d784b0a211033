"""Model zoo."""
from . import llama
from .llama import LlamaConfig, LlamaModel, LlamaForCausalLM, LlamaDecoderLayer

__all__ = ["llama", "LlamaConfig", "LlamaModel", "LlamaForCausalLM", "LlamaDecoderLayer"]
