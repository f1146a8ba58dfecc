"""Configuration: typed model configs, the architecture registry, engine-side settings."""
from .model_config import ConfigError, LlamaConfig, ModelConfig, read_config_json
from .registry import (ArchitectureEntry, config_from_dict, get_architecture, load_config,
                       register_architecture, registered_architectures)
from .engine_config import (EngineConfig, KVManagerConfig, SchedulerConfig, canonical_dtype)

__all__ = [
    "ConfigError", "LlamaConfig", "ModelConfig", "read_config_json", "ArchitectureEntry",
    "config_from_dict", "get_architecture", "load_config", "register_architecture",
    "registered_architectures", "EngineConfig", "KVManagerConfig", "SchedulerConfig",
    "canonical_dtype",
]
