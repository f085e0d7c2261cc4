"""Checkpoint formats, weight loaders and tokenizers."""
from .dptc import Checkpoint
