"""Errors a caller can tell apart by type."""


class ConfigError(ValueError):
    """config.json lacks a key, has a value of the wrong type, or names something unsupported."""


class WeightsError(ValueError):
    """A model folder's tensors do not match what the model needs."""


class CacheError(RuntimeError):
    """A slot or page of the cache was asked for that cannot be given, or given back twice."""
