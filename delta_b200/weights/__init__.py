from .loader import WeightError, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors
