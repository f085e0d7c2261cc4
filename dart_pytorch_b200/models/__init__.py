"""Model families (reference: lib/core/nn/{gpt,llama,...}.dart)."""
from .gpt import GPT, GPTConfig
