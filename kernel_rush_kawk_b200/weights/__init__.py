"""Checkpoint reading by tensor name, and seeded random weights."""

from .loader import WeightError, read_checkpoint, stored_dtype
from .random_init import random_tensor, random_tensors, write_model_folder

__all__ = ["WeightError", "read_checkpoint", "stored_dtype", "random_tensor", "random_tensors", "write_model_folder"]
