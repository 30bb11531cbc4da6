"""Architectures.  Importing this package registers them."""
from . import givirax, qwen3  # noqa: F401
