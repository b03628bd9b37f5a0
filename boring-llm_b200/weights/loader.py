"""Weights by tensor name: checked against what the model's parts declare, then handed to them.

Role of `find_tensor` / `load_model` (src/model.br:224-228, 614-690): exact-name lookup with
`tensor not found: {name}`. Added here: every problem of a checkpoint (missing names, names nobody
asked for, wrong shapes, unusable dtypes) is collected into ONE error, and shapes are checked
against the configuration, which the reference does not do.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, open_model_files, write_safetensors

# what a tensor is, which decides how the random-weights mode fills it
MATRIX, NORM, BIAS, INT_TABLE = "matrix", "norm", "bias", "int_table"


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    kind: str = MATRIX          # MATRIX | NORM | BIAS | INT_TABLE


class WeightsError(ValueError):
    """One report of everything that is wrong with a checkpoint."""


def _keep_dtype(name: str, t: torch.Tensor, spec: TensorSpec) -> torch.Tensor:
    """bfloat16 stays bfloat16, 32-bit floats stay 32-bit, half precision is widened exactly to
    32-bit, integer tables become int32."""
    if spec.kind == INT_TABLE:
        if t.dtype.is_floating_point:
            raise WeightsError(f"tensor {name}: an integer table is stored as {t.dtype}")
        return t.to(torch.int32)
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype in (torch.float16, torch.float64):
        return t.to(torch.float32)
    raise WeightsError(f"tensor {name}: unsupported dtype {t.dtype} for a weight")


def load_checkpoint(model_dir: str, expected: Dict[str, TensorSpec],
                    ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Returns `{name: CPU tensor}` for exactly the expected names.

    `ignorable` names may be present without being asked for (a stored copy of a tied output
    head, for instance). Anything else that is missing, unexpected, of the wrong shape or of an
    unusable dtype is listed in a single `WeightsError`.
    """
    try:
        files = open_model_files(model_dir)
    except SafetensorsError as e:
        raise WeightsError(str(e)) from e
    ignorable = set(ignorable)
    missing = sorted(n for n in expected if n not in files)
    unexpected = sorted(n for n in files if n not in expected and n not in ignorable)
    wrong_shape, wrong_dtype = [], []
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if name not in files:
            continue
        dtype, shape = files[name].info(name)
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append(f"{name}: file has {list(shape)}, configuration needs {list(spec.shape)}")
            continue
        try:
            out[name] = _keep_dtype(name, files[name].tensor(name), spec)
        except WeightsError as e:
            wrong_dtype.append(str(e))
    if missing or unexpected or wrong_shape or wrong_dtype:
        lines = [f"{model_dir}: the checkpoint does not match the configuration"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if wrong_dtype:
            lines.append(f"  wrong dtypes ({len(wrong_dtype)}): " + "; ".join(wrong_dtype))
        raise WeightsError("\n".join(lines))
    return out


def write_model_folder(model_dir: str, config_dict: dict, tensors) -> None:
    """config.json and model.safetensors from a configuration and a mapping `{name: tensor}`."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=2)
        f.write("\n")
    write_safetensors(os.path.join(model_dir, "model.safetensors"), {k: tensors[k].cpu() for k in tensors}, {"format": "pt"})
