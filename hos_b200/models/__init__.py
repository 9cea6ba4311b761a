"""Architectures.  Importing this package registers them."""
from . import gemma2, satapel, vagonex  # noqa: F401
