from . import dezolorn, llama  # registers Dezolorn and LlamaForCausalLM

__all__ = ["dezolorn", "llama"]
