"""Architectures: each module maps its config.json to a ``ModelSpec`` and registers itself by name."""
from . import nanbeige      # noqa: F401
