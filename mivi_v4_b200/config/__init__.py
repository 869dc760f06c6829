from .errors import ConfigError
from .lfm2 import Lfm2Config, read_config_json
from .puzorax import PuzoraxConfig
from .ropelix import RopelixConfig
from .tevirax import TeviraxConfig
from .votavik import VotavikConfig
from .registry import Architecture, architecture_for, known_architectures, register_architecture

__all__ = ["ConfigError", "Lfm2Config", "PuzoraxConfig", "RopelixConfig", "TeviraxConfig", "VotavikConfig", "read_config_json", "Architecture", "architecture_for",
           "known_architectures", "register_architecture"]
