from .loader import Checkpoint, SurplusTensorWarning, TensorWant, WeightError, device_dtype
from .random_init import RandomSource, random_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors, write_safetensors_lazy

__all__ = ["Checkpoint", "TensorWant", "WeightError", "SurplusTensorWarning", "device_dtype", "RandomSource", "random_tensor",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors", "write_safetensors_lazy"]
