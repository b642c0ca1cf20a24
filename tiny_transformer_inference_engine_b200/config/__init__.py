from .model_config import ModelConfig, ConfigError, DEFAULT_ARCHITECTURE
from .munevik_config import MunevikConfig
from .mizupel_config import MizupelConfig
from .mokalorn_config import MokalornConfig
from .dabilorn_config import DabilornConfig
from .engine_config import CacheConfig, SchedulerConfig, EngineConfig, COMPUTE_DTYPES

__all__ = ["ModelConfig", "MunevikConfig", "MizupelConfig", "MokalornConfig", "DabilornConfig", "ConfigError", "DEFAULT_ARCHITECTURE", "CacheConfig", "SchedulerConfig",
           "EngineConfig", "COMPUTE_DTYPES"]
