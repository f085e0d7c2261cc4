"""Checkpoint formats, weight loaders and tokenizers."""
from .dptc import Checkpoint
from .hf_loaders import GPT2HFLoader, LlamaHFLoader, LoadReport
from .hf_loaders_more import PythiaHFLoader, GPTJHFLoader, BertHFLoader, ClipHFLoader
from .safetensors import SafeTensors

# One report type serves every loader; the per-family names of the reference resolve to it
# (lib/core/nn/*_hf_loader.dart: GPT2LoadReport, LlamaLoadReport, PythiaLoadReport, GPTJLoadReport, BertLoadReport,
# ClipLoadReport all carry consumedCount / unusedKeys / missingKeys).
GPT2LoadReport = LlamaLoadReport = PythiaLoadReport = GPTJLoadReport = BertLoadReport = ClipLoadReport = LoadReport
