from .model_config import ConfigError, ModelConfig, read_raw_config
from .registry import ARCHITECTURES, Architecture, get_architecture, load_config, register_architecture

__all__ = ["ConfigError", "ModelConfig", "read_raw_config", "ARCHITECTURES", "Architecture",
           "get_architecture", "load_config", "register_architecture"]
