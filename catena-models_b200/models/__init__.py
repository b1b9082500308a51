"""Architectures.  Importing this package registers them by name."""
from . import lfm3  # noqa: F401
