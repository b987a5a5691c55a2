from .llama import LlamaConfig, LlamaModel, llama_local_to_hf_name

__all__ = ["LlamaConfig", "LlamaModel", "llama_local_to_hf_name"]
