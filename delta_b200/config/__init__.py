from .engine_config import EngineConfig
from .selective_cache import SelectiveCacheConfig
from .model_config import ConfigError, YiConfig
from .registry import ARCHITECTURES, Architecture, architecture_of, read_config, register_architecture, unregister_architecture
