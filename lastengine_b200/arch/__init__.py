"""Architectures the library knows.  Importing registers them."""
from . import kisilix, lenesun, lfm3, tevilix, zekivik  # noqa: F401
