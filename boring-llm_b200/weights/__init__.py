from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors, open_model_files
from .loader import (TensorSpec, WeightsError, load_checkpoint, random_tensors, write_model_folder,
                     MATRIX, NORM, BIAS, INT_TABLE)

__all__ = [
    "SafetensorsError", "SafetensorsFile", "write_safetensors", "open_model_files", "TensorSpec",
    "WeightsError", "load_checkpoint", "random_tensors", "write_model_folder",
    "MATRIX", "NORM", "BIAS", "INT_TABLE",
]
