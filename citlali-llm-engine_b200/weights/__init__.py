from .loader import TensorSpec, WeightHandle, WeightLoader
from .random_init import random_tensor, random_weights, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors
