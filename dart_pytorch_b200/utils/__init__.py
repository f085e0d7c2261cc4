"""Training utilities: flat parameter arena, CUDA-graph trainer, assignment solver."""
from .hungarian import HungarianAlgorithm
