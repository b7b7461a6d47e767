from .model_config import OPTConfig, ConfigError
from .vononex_config import VononexConfig
from .pifelix_config import PifelixConfig
from .tutelix_config import TutelixConfig
from .vozirax_config import VoziraxConfig
from .engine_config import EngineConfig, canonical_dtype
from .registry import (Architecture, register_architecture, resolve_architecture, architectures,
                       load_config, config_from_dict)
from .generation_config import (BlkSparseAttnConfig, ContinuousBatchingConfig, GenerationConfig, NeuronConfig,
                                SlidingWindowAttnConfig, SparseAttnConfig)
