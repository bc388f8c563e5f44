"""Model families owned by the framework (HF-compatible parameter names)."""
from .gpt2 import GPT2Config, GPT2LMHeadModel
from .layers import adapters_disabled, Embedding, LayerNorm, Linear, RMSNorm, linear_cross_entropy
from .llama import LlamaConfig, LlamaForCausalLM, shift_labels
from .moe import MoEConfig, MoEForCausalLM

__all__ = ["Embedding", "GPT2Config", "GPT2LMHeadModel", "LayerNorm", "Linear", "LlamaConfig", "LlamaForCausalLM", "MoEConfig", "MoEForCausalLM",
           "RMSNorm", "adapters_disabled", "linear_cross_entropy", "shift_labels"]
