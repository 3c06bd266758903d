"""Architectures the library knows.  Importing registers them."""
from . import lenesun, lfm3, zekivik  # noqa: F401
