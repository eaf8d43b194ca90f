from .base import (ConfigError, ModelConfig, config_from_dict, load_config, lookup_architecture,  # noqa: F401
                   register_architecture, registered_architectures)
from .falcon_h1 import FalconH1Config  # noqa: F401
from .turevik import TurevikConfig  # noqa: F401
from .porarax import PoraraxConfig  # noqa: F401
from .sogazen import SogazenConfig  # noqa: F401
from .kimutar import KimutarConfig  # noqa: F401
