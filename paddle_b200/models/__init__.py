"""Model families built on the framework's own layers."""
from .gpt import GPTConfig, GPTForCausalLM  # noqa: F401
from .llama import LlamaConfig, LlamaForCausalLM  # noqa: F401


def __getattr__(name):
    if name in ("MixtralConfig", "MixtralForCausalLM"):
        from . import mixtral
        return getattr(mixtral, name)
    if name == "LlamaForCausalLMInference":
        from .llama_infer import LlamaForCausalLMInference
        return LlamaForCausalLMInference
    raise AttributeError(name)
