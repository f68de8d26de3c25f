"""Checkpoints: the safetensors container, binding by name, random weights."""
from .loader import TensorSpec, check_manifest, load_tensors, stored_dtype
from .safetensors_io import SafetensorsFile, TensorStore, WeightsError, write_safetensors
