"""Tokenizers and datasets (reference: lib/core/data/*.dart)."""
from .tokenizers import CharTokenizer, BpeTokenizer
from .datasets import (Dataset, ListDataset, DataLoader, LmSample, TextEncoder, TextTokenDataset, CsvSample, CsvDataset)
from .image_folder import ImageFolderDataset, FaceSample, TripletSample
from .hf_tokenizers import HFBpeTokenizer, WordPieceTokenizer, debug_preview, debugPreview
