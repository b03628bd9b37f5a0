"""From a model folder (config.json + safetensors) to a model on the device, and the
random-weights mode that writes such a folder from a configuration and a seed."""
from __future__ import annotations

from typing import Tuple

import torch

from ..config import load_config, resolve_architecture, read_config_json
from ..weights import load_checkpoint, random_tensors, write_model_folder

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def torch_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in _DTYPES.values():
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[{"bf16": "bfloat16", "fp32": "float32", "f32": "float32"}.get(name, name)]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {name!r}") from None


def build_model(config):
    """The architecture's model for a typed configuration, weights not yet loaded."""
    arch = resolve_architecture({"architectures": [config.architecture]})
    return arch.build(config)


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> Tuple[object, object]:
    """(configuration, model on the device). The model class is chosen by config.json."""
    d = read_config_json(model_dir)
    arch = resolve_architecture(d)
    config = arch.config_cls.from_dict(d)
    model = arch.build(config)
    tensors = load_checkpoint(model_dir, model.tensor_specs(), getattr(model, "ignorable_tensors", ()))
    model.load(tensors, torch_dtype(dtype), torch.device(device))
    return config, model


def write_random_model(model_dir: str, config, seed: int, dtype="bfloat16", std: float = 0.02) -> None:
    """Writes config.json and model.safetensors of a randomly initialised model: matrices N(0, std),
    norm weights 1 + N(0, std), biases N(0, std), stored as `dtype`. The same tensors, bit for bit, as
    `load_random_model` puts on the device without a file."""
    model = build_model(config)
    tensors = random_tensors(model.tensor_specs(), seed, torch_dtype(dtype), std,
                             vocab_size=getattr(config, "vocab_size", 0))
    write_model_folder(model_dir, config.to_dict(), tensors)


def load_random_model(config, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02, weight_dtype=None):
    """(configuration, model on the device) with seeded random weights made on the device, tensor by tensor,
    without a file: what `write_random_model(dir, config, seed, weight_dtype, std)` followed by
    `load_model(dir, dtype, device)` gives, for models of any size. `weight_dtype` (default: `dtype`) is the
    type the values are rounded to before the engine takes them: "bfloat16" under a float32 engine gives the
    bfloat16 model's exact weights widened to 32-bit, which separates the rounding of weights from that of
    activations."""
    model = build_model(config)
    dev = torch.device(device)
    tensors = random_tensors(model.tensor_specs(), seed, torch_dtype(dtype if weight_dtype is None else weight_dtype),
                             std, vocab_size=getattr(config, "vocab_size", 0), device=dev)
    model.load(tensors, torch_dtype(dtype), dev)
    return config, model
