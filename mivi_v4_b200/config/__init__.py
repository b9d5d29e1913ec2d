from .errors import ConfigError
from .lfm2 import Lfm2Config, read_config_json
from .registry import Architecture, architecture_for, known_architectures, register_architecture

__all__ = ["ConfigError", "Lfm2Config", "read_config_json", "Architecture", "architecture_for",
           "known_architectures", "register_architecture"]
