"""A single-GPU inference engine for the dense Qwen2 decoder on NVIDIA B200 (sm_100a):
typed configuration and registry, safetensors weights, layers built from parts, a paged cache
manager, one step function over mixed batches, a scheduler, sampling, and hand-written CUDA kernels.
"""
from .config import (ConfigError, EngineOptions, Qwen2Config, load_config, register_architecture,
                     registered_architectures)
from .weights import WeightsError
from .models import build_model, load_model, load_random_model, write_random_model

__version__ = "0.1.0"


def __getattr__(name):
    # the engine needs torch.cuda; import it only when asked for
    if name in ("Engine", "generate", "SamplingParams", "Request", "ModelRunner", "StepEntry", "Scheduler"):
        from . import engine as _engine
        return getattr(_engine, name)
    raise AttributeError(name)
