from .loader import bind_tensors, kept_dtype, load_into
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsFile, write_safetensors
