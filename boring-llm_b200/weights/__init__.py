from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors, open_model_files
from .loader import (TensorSpec, WeightsError, load_checkpoint, write_model_folder,
                     MATRIX, NORM, BIAS, INT_TABLE)
from .random_init import RandomTensors, random_tensor, tensor_key


def random_tensors(expected, seed, dtype=None, std=0.02, vocab_size=0, device="cpu") -> RandomTensors:
    """Seeded random weights for the tensors that a model declares, as a mapping that makes each tensor when it
    is asked for (see `random_init`): matrices N(0, std), norm weights 1 + N(0, std), biases N(0, std)."""
    import torch
    return RandomTensors(expected, seed, torch.bfloat16 if dtype is None else dtype, std, vocab_size, device)


__all__ = [
    "SafetensorsError", "SafetensorsFile", "write_safetensors", "open_model_files", "TensorSpec",
    "WeightsError", "load_checkpoint", "random_tensors", "random_tensor", "tensor_key", "RandomTensors",
    "write_model_folder", "MATRIX", "NORM", "BIAS", "INT_TABLE",
]
