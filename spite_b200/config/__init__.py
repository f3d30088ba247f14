from .specs import BlockSpec, ConfigError, JunctionCall, LayerCall, ModelPlan, PartSpec, WeightBinding
from .registry import (config_class_for, config_from_dict, known_architectures, load_config,
                       register_architecture)
from .llama4 import Llama4Config, RopeScaling
from .sezazen import SezazenConfig
from .mibezen import MibezenConfig
from .paposun import PaposunConfig
from .gapevik import GapevikConfig

__all__ = ["BlockSpec", "ConfigError", "JunctionCall", "LayerCall", "ModelPlan", "PartSpec", "config_class_for",
           "config_from_dict", "known_architectures", "load_config", "register_architecture",
           "Llama4Config", "RopeScaling", "SezazenConfig", "MibezenConfig", "PaposunConfig", "GapevikConfig", "WeightBinding"]
