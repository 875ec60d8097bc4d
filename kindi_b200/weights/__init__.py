from .loader import WeightError, load_tensors
from .safetensors_io import SafetensorsError, SafetensorsFile, write_file
