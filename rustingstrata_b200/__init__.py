"""rustingstrata_b200: a small, whole inference engine for one B200 (sm_100a).

Everything between a request's token ids and its next token for the Qwen3 dense
decoder, with the capabilities of RustingStudio/RustingStrata's engine: typed
configuration and architecture registry, safetensors weights, layers assembled from
parts, a paged key/value cache, one step function for mixed prefill/decode batches, a
continuous-batching scheduler, greedy and temperature sampling, and hand-written CUDA
kernels in a bfloat16 and a true 32-bit path.
"""
from .config import EngineConfig, ConfigError, Qwen3Config  # noqa: F401
from . import models  # noqa: F401  (registers the architecture)

__version__ = "0.1.0"


def __getattr__(name):
    # the engine classes import torch and the kernel launchers; load them on first use
    if name in ("Engine", "ModelRunner", "StepEntry", "Scheduler", "Request"):
        from . import engine as _e
        return getattr(_e, name)
    if name in ("SamplingParams", "Sampler"):
        from . import sampling as _s
        return getattr(_s, name)
    raise AttributeError(name)
