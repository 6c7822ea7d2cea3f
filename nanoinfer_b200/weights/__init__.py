from .loader import WeightError, check_tensors, load_weights
from .plan import PlannedTensor, tensor_plan
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, write_safetensors

__all__ = ["WeightError", "check_tensors", "load_weights", "PlannedTensor", "tensor_plan",
           "random_tensors", "write_random_model", "SafetensorsError", "write_safetensors"]
