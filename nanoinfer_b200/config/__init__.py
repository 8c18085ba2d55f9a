from .model_config import (ConfigError, ModelConfig, Qwen2Config, read_config_json,
                           write_config_json, read_rope_theta)
from .engine_config import EngineConfig
from .kernel_options import KernelOptions

__all__ = ["ConfigError", "ModelConfig", "Qwen2Config", "EngineConfig", "read_config_json",
           "write_config_json", "read_rope_theta"]
