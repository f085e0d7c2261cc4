"""Checkpoint formats, weight loaders and tokenizers."""
from .dptc import Checkpoint
from .hf_loaders import GPT2HFLoader, LlamaHFLoader, LoadReport
from .hf_loaders_more import PythiaHFLoader, GPTJHFLoader, BertHFLoader, ClipHFLoader
from .safetensors import SafeTensors
