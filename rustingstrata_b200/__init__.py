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
