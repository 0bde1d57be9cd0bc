from .llama import ConfigError, LlamaConfig
from .registry import (Architecture, known_architectures, load_config, read_config_json,
                       register_architecture, resolve_architecture)
from .engine import EngineConfig
from .fidolix import FidolixConfig
from .kedelorn import KedelornConfig
from .povusun import PovusunConfig
from .zepavik import ZepavikConfig

__all__ = ["ConfigError", "LlamaConfig", "ZepavikConfig", "PovusunConfig", "KedelornConfig", "FidolixConfig", "EngineConfig", "Architecture", "known_architectures",
           "load_config", "read_config_json", "register_architecture", "resolve_architecture"]
