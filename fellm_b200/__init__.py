"""fellm_b200: a small, whole inference engine for the LFM2 ShortConv hybrid on one B200."""
from .config import (CacheError, ConfigError, EngineOptions, FellmError, KernelError, SchedulerError,
                     WeightError)

__all__ = ["CacheError", "ConfigError", "EngineOptions", "FellmError", "KernelError", "SchedulerError",
           "WeightError", "Engine", "GenParams"]


def __getattr__(name):
    if name in ("Engine", "GenParams", "GenStats"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)
