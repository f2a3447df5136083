"""Weights: safetensors loader by tensor name, and the random-weights mode."""
from .loader import WeightError, checkpoint_index, load_tensors
from .random import expected_tensors, random_tensors, write_random_model

__all__ = ["WeightError", "checkpoint_index", "load_tensors", "expected_tensors", "random_tensors", "write_random_model"]
