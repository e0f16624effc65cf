"""Decoder language models over `TransformerBlock` (reference: python/mojolearn/models/)."""
from .causal_lm import CausalLM, CausalLMConfig, CausalLMState  # noqa: F401
