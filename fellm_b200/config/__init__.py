from .errors import (CacheError, ConfigError, FellmError, KernelError, SchedulerError,
                     WeightError)
from .lfm2 import Lfm2Config, adjusted_ff_dim
from .options import EngineOptions
from .registry import (Architecture, architectures, config_from_dict, get_architecture,
                       read_model_config, register_architecture)
