from .engine_config import EngineConfig, parse_dtype
from .model_config import ConfigError, ModelConfig, Qwen3Config
from .registry import (build_model_spec, known_architectures, load_model_config, lookup,
                       register_model, unregister_model)

__all__ = ["EngineConfig", "parse_dtype", "ConfigError", "ModelConfig", "Qwen3Config", "build_model_spec",
           "known_architectures", "load_model_config", "lookup", "register_model", "unregister_model"]
