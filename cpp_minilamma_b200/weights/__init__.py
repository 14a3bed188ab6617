from .loader import WeightError, check_tensors, load_tensors, placement_dtype
from .random_init import random_tensors, write_random_model
from .safetensors_io import ModelFiles, SafetensorsFile, WeightFileError, write_safetensors
