from .model_config import (ConfigError, LayerCall, LayerSpec, ModelPlan, PartSpec,
                           read_config_json)
from .engine_options import EngineOptions

__all__ = ["ConfigError", "LayerCall", "LayerSpec", "ModelPlan", "PartSpec",
           "read_config_json", "EngineOptions"]
