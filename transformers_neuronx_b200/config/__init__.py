from .model_config import OPTConfig, ConfigError
from .engine_config import EngineConfig, canonical_dtype
from .registry import (Architecture, register_architecture, resolve_architecture, architectures,
                       load_config, config_from_dict)
from .generation_config import (BlkSparseAttnConfig, ContinuousBatchingConfig, GenerationConfig, NeuronConfig,
                                SlidingWindowAttnConfig, SparseAttnConfig)
