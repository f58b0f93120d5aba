"""Architectures the library knows.  Importing registers them."""
from . import lfm3  # noqa: F401
