from lily_b200.config.model_config import ConfigError, DenseDecoderConfig, RopeScaling, read_model_dir
from lily_b200.config.registry import (Architecture, register_architecture, resolve_architecture,
                                       supported_architectures)
from lily_b200.config.server_args import ServerArgs

__all__ = ["ConfigError", "DenseDecoderConfig", "RopeScaling", "read_model_dir", "Architecture",
           "register_architecture", "resolve_architecture", "supported_architectures", "ServerArgs"]
