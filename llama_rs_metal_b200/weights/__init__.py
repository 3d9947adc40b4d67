from .loader import TensorSpec, canonical_name, check_names_and_shapes, load_tensors
from .random_init import random_tensors, write_model_folder
from .safetensors_io import TensorEntry, open_checkpoint, write_safetensors

__all__ = ["TensorSpec", "canonical_name", "check_names_and_shapes", "load_tensors",
           "random_tensors", "write_model_folder", "TensorEntry", "open_checkpoint",
           "write_safetensors"]
