"""Model definitions used by the end-to-end data-parallel runs."""
from .llama import LlamaConfig, LlamaForCausalLM  # noqa: F401
