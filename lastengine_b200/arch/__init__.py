"""Architectures the library knows.  Importing registers them."""
from . import lfm3, zekivik  # noqa: F401
