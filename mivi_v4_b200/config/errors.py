"""Errors raised while reading a model's configuration."""


class ConfigError(ValueError):
    """A config.json that is missing a key, has a value of the wrong kind, or
    describes sizes that do not fit together."""
