from .engine_config import DEFAULT_PAGE_SIZE, EngineConfig, parse_dtype
from .model_config import ConfigError, Qwen2VLConfig, read_config_dict
from .registry import known_architectures, register_architecture, resolve, resolve_dir
