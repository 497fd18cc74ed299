"""Weights: safetensors reading and writing, name resolution with one clear error, random init."""
from .loader import check_names_and_shapes, load_into  # noqa: F401
from .random_init import init_random, random_tensor, write_random_model  # noqa: F401
from .safetensors_io import SafetensorsFile, open_model_files, save_safetensors  # noqa: F401
