from .model_config import ConfigError, LlamaConfig, ModelConfig, RopeScaling, read_config_json
from .deganex_config import DeganexConfig
from .lotirax_config import LotiraxConfig
from .tubazen_config import TubazenConfig
from .lugizen_config import LugizenConfig
from .registry import (architecture_of, load_config, lookup_architecture, register_architecture,
                       registered_architectures, unregister_architecture)
