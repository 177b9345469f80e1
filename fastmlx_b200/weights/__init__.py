from .loader import WeightError, load_checkpoint, load_tensors, shard_files
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = ["WeightError", "load_checkpoint", "load_tensors", "shard_files",
           "random_tensor", "random_tensors", "write_random_model"]
