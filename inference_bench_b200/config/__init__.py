"""Typed configurations, one module per architecture."""


class ConfigError(ValueError):
    """config.json cannot be turned into a model of a registered architecture."""
