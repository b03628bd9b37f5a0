"""Builds the CUDA sources under `csrc/` into one shared library for sm_100a and loads it.

The library is built in the tree (`csrc/_build/libboring_b200.so`) the first time it is needed and
again whenever a source, a header or a flag changes; if the tree cannot be written, a folder under
the system's temporary directory is used. There is no other implementation behind these kernels:
if the library cannot be built or loaded, or the device is not a compute-capability-10 GPU, using it
raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
_LIB_NAME = "libboring_b200.so"
_NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "--compiler-options", "-fPIC", "--expt-relaxed-constexpr",
]

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


class KernelLibraryError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelLibraryError("nvcc not found (set CUDA_HOME or NVCC): the CUDA kernels cannot be built")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(_CSRC) if f.endswith(".cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(_NVCC_FLAGS).encode())
    for f in sorted(os.listdir(_CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(_CSRC, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.path.join(_CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"boring_llm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path() -> str:
    return os.path.join(_build_dir(), _LIB_NAME)


def build(verbose: bool = True, force: bool = False) -> str:
    """Compiles what is stale and links the library; returns its path."""
    bdir = _build_dir()
    lib = os.path.join(bdir, _LIB_NAME)
    stamp = os.path.join(bdir, "fingerprint.txt")
    fp = _fingerprint()
    if not force and os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == fp:
                return lib
    nvcc = _nvcc()
    srcs = sources()
    t0 = time.time()

    def say(msg):
        if verbose:
            print(f"[boring-llm_b200] {msg}", file=sys.stderr, flush=True)

    say(f"building {len(srcs)} CUDA sources for sm_100a in {bdir} (first use or sources changed)")

    def compile_one(src):
        obj = os.path.join(bdir, src[:-3] + ".o")
        cmd = [nvcc] + _NVCC_FLAGS + ["-I", _CSRC, "-c", os.path.join(_CSRC, src), "-o", obj]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise KernelLibraryError(f"nvcc failed on {src}:\n{p.stdout}")
        say(f"compiled {src} ({time.time() - t0:.0f} s)")
        return obj

    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            say(f"still compiling ... {time.time() - t0:.0f} s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        with ThreadPoolExecutor(max_workers=min(8, max(1, os.cpu_count() or 1))) as ex:
            objs = list(ex.map(compile_one, srcs))
        tmp = lib + f".{os.getpid()}.tmp"
        cmd = [nvcc, "-shared", "-o", tmp] + objs + ["-lcudart"]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise KernelLibraryError(f"linking {_LIB_NAME} failed:\n{p.stdout}")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(fp + "\n")
    finally:
        done.set()
    say(f"built {_LIB_NAME} in {time.time() - t0:.0f} s")
    return lib


def load() -> ctypes.CDLL:
    """The loaded library (built first if needed)."""
    global _lib
    if _lib is not None:                       # the common case, hundreds of times a step: no lock
        return _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelLibraryError(f"cannot load {path}: {e}") from e
            _lib.bl_last_error.restype = ctypes.c_char_p
        return _lib
