from .specs import BlockSpec, ConfigError, LayerCall, ModelPlan, PartSpec
from .registry import (config_class_for, config_from_dict, known_architectures, load_config,
                       register_architecture)
from .llama4 import Llama4Config, RopeScaling, WeightBinding

__all__ = ["BlockSpec", "ConfigError", "LayerCall", "ModelPlan", "PartSpec", "config_class_for",
           "config_from_dict", "known_architectures", "load_config", "register_architecture",
           "Llama4Config", "RopeScaling", "WeightBinding"]
