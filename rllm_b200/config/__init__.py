from .base import (Architecture, ConfigError, ModelConfig, config_from_dict, load_config,
                   register_architecture, registered_architectures, resolve_architecture)
from .llama import LlamaConfig, RopeScaling
from .livovik import LivovikConfig, LivovikLayer, LivovikMLP, SinkAttentionConfig
from .bazulorn import BazulornConfig, BazulornLayer, BazulornMLP
from .purozen import PurozenConfig, PurozenLayer
from .zukotar import GLAConfig, LatentAttentionConfig, MoEConfig, ZukotarConfig

__all__ = ["Architecture", "ConfigError", "ModelConfig", "config_from_dict", "load_config",
           "register_architecture", "registered_architectures", "resolve_architecture",
           "LlamaConfig", "RopeScaling", "GLAConfig", "LatentAttentionConfig", "MoEConfig", "ZukotarConfig",
           "LivovikConfig", "LivovikLayer", "LivovikMLP", "SinkAttentionConfig",
           "BazulornConfig", "BazulornLayer", "BazulornMLP", "PurozenConfig", "PurozenLayer"]
