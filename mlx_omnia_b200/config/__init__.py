"""Typed configurations and their hydration from config.json."""

from mlx_omnia_b200.config.hydrate import ConfigError, hydrate, read_json

__all__ = ["ConfigError", "hydrate", "read_json"]
