from .base import ConfigError, ModelConfig, read_config_json
from .lfm2 import Lfm2Config
from .registry import (architecture_name, build_model, config_from_dict, config_from_folder, get_architecture,
                       register_architecture, registered_architectures, unregister_architecture)
