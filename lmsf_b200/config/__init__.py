from .engine_config import CacheConfig, EngineArgs, SchedulerConfig, canonical_dtype, resolve_max_model_len
from .model_config import ConfigError, LlamaConfig, RopeScaling, read_config_json
from .registry import (load_model_config, register_architecture, registered_architectures, resolve_architecture)
