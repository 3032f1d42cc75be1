"""Model families built on the framework's own layers."""
from .gpt import GPTConfig, GPTForCausalLM  # noqa: F401
from .llama import LlamaConfig, LlamaForCausalLM  # noqa: F401
