"""Benchmark and test models (stock PyTorch forward / backward)."""

from .gpt2 import GPT2, GPT2Config
from .llama import Llama, LlamaConfig, num_params
from .mlp import make_mlp

__all__ = ["GPT2", "GPT2Config", "Llama", "LlamaConfig", "make_mlp", "num_params"]
