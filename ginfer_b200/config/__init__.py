from .engine_config import EngineConfig
from .model_config import ConfigError, Qwen2Config, read_config_json
from .vilepel_config import VilepelConfig, VilepelLayer
from .registry import (load_model_config, register_architecture, registered_architectures,
                       resolve_architecture)
