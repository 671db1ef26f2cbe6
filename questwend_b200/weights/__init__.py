from .manifest import TensorSpec, MATRIX, VECTOR, TABLE, NORMAL, NORM_WEIGHT
from .safetensors_io import SafetensorsFile, SafetensorsFolder, SafetensorsError, write_safetensors
from .loader import WeightsError, check_manifest, load_tensors, held_dtype
from .random_init import random_tensors, write_model_folder

__all__ = ["TensorSpec", "MATRIX", "VECTOR", "TABLE", "NORMAL", "NORM_WEIGHT", "SafetensorsFile",
           "SafetensorsFolder", "SafetensorsError", "write_safetensors", "WeightsError",
           "check_manifest", "load_tensors", "held_dtype", "random_tensors", "write_model_folder"]
