"""Typed configurations, one class per architecture, read from ``config.json``."""

from tokenomos_b200.config.lfm3 import ConfigError, Lfm3Config, RopeParams

__all__ = ["ConfigError", "Lfm3Config", "RopeParams"]
