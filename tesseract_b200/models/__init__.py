from .llama import GenerateConfig, LlamaConfig, LlamaModel, llama_local_to_hf_name
from .sampler import MT19937_64, Sampler, SamplingParams, sample_from_logits

__all__ = ["GenerateConfig", "LlamaConfig", "LlamaModel", "llama_local_to_hf_name", "MT19937_64", "Sampler",
           "SamplingParams", "sample_from_logits"]
