"""Weights: safetensors files by tensor name, checked loading, and seeded random weights."""
from .safetensors_io import SafetensorsError, SafetensorsFile, TensorSource, write_safetensors
from .loader import TensorWant, WeightError, compare, convert_checked, load_checked, target_dtype
from .random_init import random_tensors, write_model_folder
