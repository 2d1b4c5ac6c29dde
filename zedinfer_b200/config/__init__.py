from .spec import PartSpec, LayerSpec, LayerCall, ModelSpec
from .registry import (Architecture, ConfigError, register_architecture, unregister_architecture,
                       resolve_architecture, supported_architectures, read_config_json, load_model_config)
from .engine_config import SchedulerConfig, GenerationConfig, resolve_max_new_tokens, sampling_defaults

__all__ = ["PartSpec", "LayerSpec", "LayerCall", "ModelSpec", "Architecture", "ConfigError",
           "register_architecture", "unregister_architecture", "resolve_architecture",
           "supported_architectures", "read_config_json", "load_model_config",
           "SchedulerConfig", "GenerationConfig", "resolve_max_new_tokens", "sampling_defaults"]
