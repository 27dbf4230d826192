"""Weights: the safetensors container, loading by name, random models."""
from .params import ParamSpec
from .safetensors_io import SafetensorsFile, write_safetensors
from .loader import check_tensors, convert, load_tensors, open_checkpoint
from .random_init import draw, random_tensors, random_tensors_on_device, write_model_folder

__all__ = ["ParamSpec", "SafetensorsFile", "write_safetensors", "check_tensors", "convert",
           "load_tensors", "open_checkpoint", "draw", "random_tensors", "random_tensors_on_device", "write_model_folder"]
