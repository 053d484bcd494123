"""Architectures: each module turns its typed configuration into a ``ModelSpec`` and
registers itself by the name found in config.json."""
from . import fekolorn, pozelix, pusazen, qwen3, rusadra

__all__ = ["fekolorn", "pozelix", "pusazen", "qwen3", "rusadra"]
