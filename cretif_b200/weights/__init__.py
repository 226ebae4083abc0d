"""Weights: the safetensors container, checked loading by name, random weights."""
from .safetensors_io import (CheckpointError, checkpoint_files, read_header, read_tensors,
                             write_tensors)
from .loader import WeightSpec, load_weights, random_weights, write_model_folder

__all__ = ["CheckpointError", "checkpoint_files", "read_header", "read_tensors", "write_tensors",
           "WeightSpec", "load_weights", "random_weights", "write_model_folder"]
