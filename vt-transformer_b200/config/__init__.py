from .base import ConfigError, KeyReader, ModelConfig
from .fosepel import FosepelConfig
from .geponex import GeponexConfig
from .qwen2 import Qwen2Config
from .sisetar import SisetarConfig
from .vegilix import VegilixConfig
from .registry import (Architecture, config_from_dict, get_architecture, known_architectures, load_config,
                       register_architecture, unregister_architecture)
