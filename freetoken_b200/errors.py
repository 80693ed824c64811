"""Exception types raised by the framework; each names what the user must fix."""


class FreeTokenError(Exception):
    """Base class of every error the framework raises on purpose."""


class ConfigError(FreeTokenError):
    """config.json (or an engine option) holds a value the engine cannot run."""


class WeightError(FreeTokenError):
    """The weight files do not match the tensors the model expects."""


class KernelError(FreeTokenError):
    """A CUDA kernel refused its arguments, or the native library is unavailable."""


class CacheError(FreeTokenError):
    """The cache manager was asked for something it cannot give (pages, slots)."""


class SchedulerError(FreeTokenError):
    """A request cannot be admitted or run."""
