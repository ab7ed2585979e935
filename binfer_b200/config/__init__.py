"""Configuration: architecture-neutral specs, family configs, and the architecture registry."""
from .specs import (AttentionSpec, ConfigError, GatedMLPSpec, LayerSpec, MLSTMSpec, ModelSpec,
                    NameLayout, NormSpec, PooledWindowAttentionSpec, RopeSpec, ScheduleEntry,
                    ScoreSpec)
from .qwen3 import Qwen3Config
from .gukidra import GukidraConfig
from .registry import (family_for, load_config, parse_config, read_config_json,
                       register_architecture, registered_architectures)

__all__ = [
    "AttentionSpec", "ConfigError", "GatedMLPSpec", "LayerSpec", "ModelSpec", "NameLayout",
    "NormSpec", "RopeSpec", "ScheduleEntry", "ScoreSpec", "Qwen3Config",
    "GukidraConfig", "MLSTMSpec", "PooledWindowAttentionSpec", "family_for", "load_config",
    "parse_config", "read_config_json", "register_architecture", "registered_architectures",
]
