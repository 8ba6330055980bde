from .loader import WeightsError, checkpoint_files, load_tensors
from .random_init import random_tensors, write_random_model

__all__ = ["WeightsError", "checkpoint_files", "load_tensors", "random_tensors", "write_random_model"]
