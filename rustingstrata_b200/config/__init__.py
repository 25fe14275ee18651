from .model_config import ConfigError, Qwen3Config, read_config_json, FULL_ATTENTION, SLIDING_ATTENTION
from .engine_config import EngineConfig
from .registry import (Architecture, register_architecture, unregister_architecture, registered_architectures,
                       resolve_architecture, load_model_config)
