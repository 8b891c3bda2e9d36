from .loader import WeightError, check_tensors, load_weights
from .random_init import init_random_on_device, write_random_model
from .safetensors_io import SafetensorsError, open_model_tensors, write_safetensors
