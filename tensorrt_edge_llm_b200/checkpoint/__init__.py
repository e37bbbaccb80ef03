"""Checkpoint reading, weight loading and load-time repacking."""
from .loader import load_weights, init_random_weights
from .safetensors_io import CheckpointReader, SafetensorsFile, save_file

__all__ = ["load_weights", "init_random_weights", "CheckpointReader", "SafetensorsFile", "save_file"]
