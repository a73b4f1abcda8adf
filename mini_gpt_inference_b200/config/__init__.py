from .engine_config import EngineConfig, SamplingParams, canonical_dtype
from .fakilorn_config import FakilornConfig
from .model_config import ConfigError, GPTConfig, read_config_json
from .lunelorn_config import LunelornConfig
from .nukodra_config import NukodraConfig
from .zenedra_config import ZenedraConfig
from .registry import (MODEL_REGISTRY, ModelFamily, UnknownArchitectureError, architecture_name,
                       load_config, lookup, register_model)

__all__ = ["EngineConfig", "SamplingParams", "canonical_dtype", "ConfigError", "FakilornConfig", "GPTConfig",
           "read_config_json", "LunelornConfig", "NukodraConfig", "ZenedraConfig", "MODEL_REGISTRY", "ModelFamily", "UnknownArchitectureError",
           "architecture_name", "load_config", "lookup", "register_model"]
