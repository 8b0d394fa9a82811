"""Architectures the library knows.  Importing registers them."""
from . import kisilix, lenesun, lfm3, zekivik  # noqa: F401
