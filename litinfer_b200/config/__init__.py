from .qwen2 import ConfigError, Qwen2Config
from .registry import (
    config_class_for,
    config_from_dict,
    load_config,
    model_spec_from_dir,
    register_architecture,
    supported_architectures,
)
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule, validate_schedule

__all__ = [
    "BlockSpec",
    "ConfigError",
    "ModelSpec",
    "PartSpec",
    "Qwen2Config",
    "ScheduleEntry",
    "config_class_for",
    "config_from_dict",
    "default_schedule",
    "load_config",
    "model_spec_from_dir",
    "register_architecture",
    "supported_architectures",
    "validate_schedule",
]
