"""The random-weights generator: every element of every tensor is a pure function of (seed, tensor name, index).

The reference has random weights only in its fixture generator, which draws tensor after tensor from one
numpy stream (tools/make_arch_test_ggufs.py:214-227): the values depend on the order of the draws and exist only
on the host. Here a tensor's values depend on nothing but the seed, the tensor's checkpoint name and the element's
flat index, so that

* a model can be built in device memory tensor by tensor without a file (a model of 15 GB need not be written
  and read back), and dumped to a model folder when one is wanted: both give the same bits;
* the order in which tensors are made, and the device they are made on, do not matter.

Bit-equality between the CPU and the GPU rules out library `log` and `cos` (their last bit differs between
implementations), so the normal deviates are made from operations that IEEE 754 defines exactly, each as a
separate tensor operation in 64-bit (no fused multiply-add can form): integer mixing, `+ - * /`, `sqrt`, and
`frexp`.

    key      = first 8 bytes (little endian) of SHA-256("{seed}:{tensor name}")
    h1       = mix(key + index * 0x9E3779B97F4A7C15)            (64-bit wrapping arithmetic)
    h2       = mix(h1 + 0xD1B54A32D192ED03)
    u        = ((h1 >> 11) + 1) / 2^53                          in (0, 1]
    k        = h2 >> 32                                         32 bits: the angle 2 pi k / 2^32
    z        = sqrt(-2 ln u) * cos(2 pi k / 2^32)               Box-Muller
    ln u     = e ln 2 + 2 (s + s^3/3 + ... + s^23/23),  u = m 2^e with m in [sqrt(1/2), sqrt(2)), s = (m - 1)/(m + 1)
    cos      = by quadrant (the top two bits of k) from the Taylor series of sin and cos on [0, pi/2), 13 terms each
    mix(x)   : x ^= x >> 32; x *= 0xD6E8FEB86659FD93; x ^= x >> 29; x *= 0xCA9B0D9B0D7E5B4F | 1; x ^= x >> 32

    matrix, bias:  value = z * std        norm weight:  value = 1 + z * std        integer table:  h1 mod vocab

computed in 64-bit, rounded once to 32-bit and once more to the storage type.
"""
from __future__ import annotations

import hashlib
import math
from collections.abc import Mapping
from typing import Dict, Iterator

import torch

from .loader import BIAS, INT_TABLE, MATRIX, NORM, TensorSpec

_M64 = (1 << 64) - 1
_STEP = 0x9E3779B97F4A7C15
_NEXT = 0xD1B54A32D192ED03
_MUL1 = 0xD6E8FEB86659FD93
_MUL2 = 0xCA9B0D9B0D7E5B4F | 1
_CHUNK = 1 << 22                 # elements made at a time: bounds the 64-bit temporaries (32 MB each)


def _s64(v: int) -> int:
    """The 64-bit pattern `v` as the signed integer that torch's int64 holds."""
    v &= _M64
    return v - (1 << 64) if v >> 63 else v


def _shr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical shift right of 64-bit patterns held in int64 (torch's >> keeps the sign)."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def _mix(x: torch.Tensor) -> torch.Tensor:
    x = x ^ _shr(x, 32)
    x = x * _s64(_MUL1)
    x = x ^ _shr(x, 29)
    x = x * _s64(_MUL2)
    return x ^ _shr(x, 32)


def tensor_key(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()[:8], "little")


def _horner(x2: torch.Tensor, coeffs) -> torch.Tensor:
    """c[0] + c[1] x2 + c[2] x2^2 + ...: one multiplication and one addition per term, each rounded by itself."""
    p = torch.full_like(x2, coeffs[-1])
    for c in reversed(coeffs[:-1]):
        p = p * x2
        p = p + c
    return p


_LN_COEFFS = [1.0 / (2 * k + 1) for k in range(12)]
_COS_COEFFS = [(-1.0) ** n / math.factorial(2 * n) for n in range(13)]
_SIN_COEFFS = [(-1.0) ** n / math.factorial(2 * n + 1) for n in range(13)]
_SQRT_HALF = math.sqrt(0.5)
_LN2 = math.log(2.0)
_QUARTER_TURN = (math.pi / 2) / float(1 << 30)


def _hashes(key: int, start: int, n: int, device) -> tuple:
    idx = torch.arange(start, start + n, dtype=torch.int64, device=device)
    h1 = _mix(idx * _s64(_STEP) + _s64(key))
    h2 = _mix(h1 + _s64(_NEXT))
    return h1, h2


def _normal_chunk(key: int, start: int, n: int, device) -> torch.Tensor:
    """Elements [start, start + n) of the standard normal stream of `key`, in 64-bit."""
    h1, h2 = _hashes(key, start, n, device)
    u = (_shr(h1, 11) + 1).to(torch.float64) * (2.0 ** -53)
    m, e = torch.frexp(u)                                   # u = m 2^e, m in [1/2, 1)
    low = m < _SQRT_HALF
    m = torch.where(low, m * 2.0, m)
    e = torch.where(low, e - 1, e).to(torch.float64)
    s = (m - 1.0) / (m + 1.0)
    ln_u = e * _LN2 + (s * _horner(s * s, _LN_COEFFS)) * 2.0
    r = torch.sqrt(ln_u * -2.0)
    k = _shr(h2, 32)
    quadrant = k >> 30
    theta = (k & ((1 << 30) - 1)).to(torch.float64) * _QUARTER_TURN
    t2 = theta * theta
    c = _horner(t2, _COS_COEFFS)
    sn = theta * _horner(t2, _SIN_COEFFS)
    # cos(q pi/2 + theta) = cos, -sin, -cos, sin for q = 0, 1, 2, 3
    w = torch.where(quadrant == 0, c, torch.where(quadrant == 1, -sn, torch.where(quadrant == 2, -c, sn)))
    return r * w


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                  vocab_size: int = 0, device="cpu") -> torch.Tensor:
    """The tensor `name` of the random model `seed`: matrices and biases N(0, std), norm weights 1 + N(0, std),
    integer tables uniform in [0, vocab_size), stored as `dtype` (integer tables as int32)."""
    device = torch.device(device)
    n = 1
    for d in spec.shape:
        n *= int(d)
    key = tensor_key(seed, name)
    out = torch.empty(n, dtype=torch.int32 if spec.kind == INT_TABLE else dtype, device=device)
    for start in range(0, n, _CHUNK):
        m = min(_CHUNK, n - start)
        if spec.kind == INT_TABLE:
            h1, _ = _hashes(key, start, m, device)
            out[start:start + m] = (_shr(h1, 1) % max(int(vocab_size), 2)).to(torch.int32)
            continue
        v = _normal_chunk(key, start, m, device) * float(std)
        if spec.kind == NORM:
            v = v + 1.0
        elif spec.kind not in (MATRIX, BIAS):
            raise ValueError(f"tensor {name}: unknown kind {spec.kind!r}")
        out[start:start + m] = v.to(torch.float32).to(dtype)
    return out.reshape(tuple(spec.shape))


class RandomTensors(Mapping):
    """`{name: tensor}` of a random model, each tensor made when it is asked for (and again when asked again):
    a model takes its tensors one by one, so that never more than one of them exists beside the placed model."""

    def __init__(self, expected: Dict[str, TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                 std: float = 0.02, vocab_size: int = 0, device="cpu"):
        self.expected, self.seed, self.dtype, self.std = dict(expected), int(seed), dtype, float(std)
        self.vocab_size, self.device = int(vocab_size), torch.device(device)

    def __getitem__(self, name: str) -> torch.Tensor:
        return random_tensor(name, self.expected[name], self.seed, self.dtype, self.std, self.vocab_size, self.device)

    def __iter__(self) -> Iterator[str]:
        return iter(sorted(self.expected))

    def __len__(self) -> int:
        return len(self.expected)
