from .model_config import ConfigError, ModelConfig, read_config_json, read_eos_token_ids, resolve_rope_theta
from .registry import (Architecture, architecture_of, check_config_protocol, register_architecture,
                       supported_architectures, unregister_architecture)

__all__ = ["Architecture", "ConfigError", "ModelConfig", "architecture_of", "check_config_protocol",
           "read_config_json", "read_eos_token_ids", "register_architecture", "resolve_rope_theta",
           "supported_architectures", "unregister_architecture"]
