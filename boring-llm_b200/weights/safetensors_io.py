"""Reader and writer for the safetensors container (own implementation, no third-party reader).

Layout of a file: 8 bytes little-endian header length N, N bytes of JSON
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`, then raw
little-endian tensor data; offsets are relative to the first byte after the header.

Role of the reference's GGUF parser (src/gguf.br:222-275, src/gguf_file.br:65-112): only the header
is parsed, each tensor is read on demand by byte range, and a hostile or truncated file gives an
error instead of a crash (src/gguf.br:36-40, 248, 257, 267; src/gguf_file.br:92).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 256 << 20
_MAX_ELEMENTS = 1 << 40


class SafetensorsFile:
    """One opened file: `names()`, `info(name)` and `tensor(name)` (a CPU tensor over the mapping)."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > _MAX_HEADER or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        raw = self._f.read(n)
        try:
            header = json.loads(raw.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + n
        data_len = size - self._data_start
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            if not isinstance(e, dict) or not {"dtype", "shape", "data_offsets"} <= set(e):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}")
            if e["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: unsupported dtype {e['dtype']!r} for tensor {name!r}")
            dtype, item = _DTYPES[e["dtype"]]
            shape = e["shape"]
            if (not isinstance(shape, list) or len(shape) > 8
                    or not all(isinstance(s, int) and s >= 0 for s in shape)):
                raise SafetensorsError(f"{path}: invalid shape {shape!r} for tensor {name!r}")
            numel = 1
            for s in shape:
                numel *= s
            if numel > _MAX_ELEMENTS:
                raise SafetensorsError(f"{path}: tensor {name!r} has too many elements ({numel})")
            off = e["data_offsets"]
            if (not isinstance(off, list) or len(off) != 2
                    or not all(isinstance(o, int) for o in off)):
                raise SafetensorsError(f"{path}: invalid data_offsets for tensor {name!r}")
            begin, end = off
            if begin < 0 or end < begin or end > data_len:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} lies outside the file (offsets {begin}..{end}, data {data_len} bytes)")
            if end - begin != numel * item:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} has {end - begin} bytes but shape {shape} of {e['dtype']} "
                    f"needs {numel * item}")
            self._entries[name] = (dtype, tuple(shape), begin, end)
        self._map = None

    def names(self):
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self._entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self._entries:
            raise SafetensorsError(f"{self.path}: tensor not found: {name}")
        dtype, shape, begin, end = self._entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        if self._map is None:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        buf = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # the mapping is read-only; tensors are copied on use
            t = torch.frombuffer(buf, dtype=dtype)
        return t.reshape(shape)

    def close(self):
        self._map = None
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Writes tensors in name order; the data section starts on an 8-byte boundary."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} (tensor {name!r})")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> Dict[str, SafetensorsFile]:
    """Maps every tensor name of a model folder to the file that holds it: `model.safetensors`,
    or the shards that `model.safetensors.index.json` lists (role of split GGUF shards,
    src/gguf.br:329-354)."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    out: Dict[str, SafetensorsFile] = {}
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        for n in f.names():
            out[n] = f
        return out
    if os.path.isfile(index):
        try:
            with open(index, "r", encoding="utf-8") as fh:
                wm = json.load(fh)["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError) as e:
            raise SafetensorsError(f"{index}: not a valid shard index ({e})") from e
        files: Dict[str, SafetensorsFile] = {}
        for name, fname in wm.items():
            if fname not in files:
                files[fname] = SafetensorsFile(os.path.join(model_dir, os.path.basename(fname)))
            if name not in files[fname].names():
                raise SafetensorsError(f"{index}: tensor {name!r} is not in shard {fname}")
            out[name] = files[fname]
        return out
    raise SafetensorsError(f"{model_dir}: no model.safetensors (or model.safetensors.index.json) in the model folder")
