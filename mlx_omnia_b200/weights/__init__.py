"""Reading checkpoints strictly by tensor name, and writing random ones."""

from mlx_omnia_b200.weights.loader import WeightError, checkpoint_files, load_tensors
from mlx_omnia_b200.weights.random_init import write_random_model

__all__ = ["WeightError", "checkpoint_files", "load_tensors", "write_random_model"]
