from .causal_lm import CausalLM
from . import qwen3  # noqa: F401  (registers the architecture)
from .manifest import manifest_for  # noqa: E402,F401
