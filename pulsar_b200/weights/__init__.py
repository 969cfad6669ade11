from .loader import WeightError, check_entries, load_weights
from .random_init import load_random, random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors
