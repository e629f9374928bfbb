"""Error types of the engine (FeLLM has one enum, crates/fellm-core/src/error.rs:7)."""


class FellmError(Exception):
    """Base of every error this package raises on purpose."""


class ConfigError(FellmError):
    """config.json is missing, malformed, or asks for something the engine cannot build."""


class WeightError(FellmError):
    """The weight file does not match the model: missing, unexpected or misshapen tensors."""


class CacheError(FellmError):
    """The cache manager cannot do what was asked (no pages left, unknown request, ...)."""


class KernelError(FellmError):
    """A CUDA kernel is missing, failed to build, refused a size, or reported a fault."""


class SchedulerError(FellmError):
    """A request cannot be accepted (too long for the context or for the page pool)."""
