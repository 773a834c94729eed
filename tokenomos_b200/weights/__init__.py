"""Model folders: reading safetensors by tensor name, and the random-weights mode."""

from tokenomos_b200.weights.checkpoint import Checkpoint, WeightError, check, load_tensors
from tokenomos_b200.weights.random_init import random_tensors, write_model_folder

__all__ = ["Checkpoint", "WeightError", "check", "load_tensors", "random_tensors",
           "write_model_folder"]
