"""Weights: safetensors by tensor name, and a random-weights mode."""

from simply_b200.weights.loader import TensorSpec, WeightError, check, load_tensors
from simply_b200.weights.random_init import random_tensors, write_model_folder

__all__ = ["TensorSpec", "WeightError", "check", "load_tensors", "random_tensors",
           "write_model_folder"]
