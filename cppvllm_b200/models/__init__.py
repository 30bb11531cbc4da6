"""Architectures.  Importing this package registers them."""
from . import dugulorn, givirax, qwen3  # noqa: F401
