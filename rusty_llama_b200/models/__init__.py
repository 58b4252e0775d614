"""Architectures.  Importing this package registers them."""

from . import llama, vezatar  # noqa: F401
