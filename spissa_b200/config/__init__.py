"""Typed configurations and the architecture registry."""
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
from .registry import (UnknownArchitecture, config_class_for, config_from_dict, known_architectures,
                       load_config, register_architecture, unregister_architecture)
from .llama import ConfigError, LlamaConfig, RopeScaling

__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule",
           "UnknownArchitecture", "config_class_for", "config_from_dict", "known_architectures",
           "load_config", "register_architecture", "unregister_architecture",
           "ConfigError", "LlamaConfig", "RopeScaling"]
