from .loader import FolderSource, RandomSource, WeightsError, check_tensors, kept_dtype, load_weights
from .random_init import write_random_model
from .safetensors_io import Deferred, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["Deferred", "FolderSource", "RandomSource", "SafetensorsError", "SafetensorsFile", "WeightsError",
           "check_tensors", "kept_dtype", "load_weights", "write_random_model", "write_safetensors"]
