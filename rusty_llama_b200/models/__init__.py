"""Architectures.  Importing this package registers them."""

from . import llama, revirax, vezatar  # noqa: F401
