from . import dezolorn, llama, sorizen  # registers Dezolorn, LlamaForCausalLM and Sorizen

__all__ = ["dezolorn", "llama", "sorizen"]
