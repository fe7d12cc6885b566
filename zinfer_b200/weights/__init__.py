from .loader import WeightError, load_model
from .random_init import random_model, write_random_model
from .safetensors_io import SafetensorsFile, WeightFileError, write_safetensors
